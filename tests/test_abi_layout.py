"""The library is called by programs compiled against the reference's headers,
so the restated structs in include/seraph_b200_abi.h must have the reference's
layout.  Compiles one probe against each header set and compares
sizeof/offsetof of every struct and every field the library uses.  Needs the
reference checkout; skipped without it."""
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout: SERAPH_REFERENCE, or a directory `reference` beside this repository
REF = os.environ.get("SERAPH_REFERENCE") or os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))

FIELDS = {
    "cuda_buffer_t": ["data", "size"],
    "cuda_lora_gpu_adapter_t": ["A", "B", "gA", "gB", "mA", "vA", "mB", "vB", "active"],
    "cuda_lora_gpu_state_t": ["num_layers", "rank", "alpha", "scale", "q", "k", "v", "o", "gate", "up", "down"],
    "cuda_train_context_t": [
        "device_id", "stream", "initialized", "gpu_sm_count", "gpu_regs_per_sm", "use_bf16", "use_flash_attn",
        "batch_size", "attention_num_warps", "weight_buffer", "max_buffer_size", "max_fwd_buffer_size",
        "max_attn_buffer_size", "fwd_hidden_buffer", "max_fwd_act_bytes", "fwd_cache_num_layers",
        "fwd_cache_x_norm_attn", "fwd_cache_attn_lse", "train_tokens_u32", "train_final_input",
        "gpu_weights_num_layers", "gpu_weights_vocab_size", "gpu_w_embed", "gpu_v_final_norm", "gpu_w_q",
        "gpu_v_q", "gpu_w_down", "gpu_v_post_norm", "debug_nan_flags", "lora_gpu", "lora_hidden_tmp",
        "lora_hidden_tmp_bytes"],
    "weight_tensor_t": ["weight", "grad", "m", "v", "size"],
    "layer_weights_t": ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj",
                        "input_norm", "post_norm"],
    "trainable_weights_t": ["num_layers", "hidden_size", "intermediate_size", "vocab_size", "layers",
                            "embed_tokens", "final_norm", "total_params"],
    "lora_adapter_t": ["in_dim", "out_dim", "rank", "alpha", "A", "B", "grad_A", "grad_B", "m_A", "v_A", "m_B", "v_B"],
    "lora_model_t": ["num_layers", "rank", "alpha", "dropout", "apply_to_q", "apply_to_ffn", "q_adapters",
                     "k_adapters", "v_adapters", "o_adapters", "gate_adapters", "up_adapters", "down_adapters"],
    "model_config_t": ["vocab_size", "hidden_size", "num_hidden_layers", "intermediate_size",
                       "num_attention_heads", "num_key_value_heads", "head_dim", "kv_dim", "rms_norm_eps",
                       "rope_theta", "max_position_embeddings", "use_qk_norm", "clip_embeddings_path",
                       "hidden_act", "tie_word_embeddings", "model_dir"],
    "train_state_t": ["model", "config", "train_cfg", "use_full_training", "lora", "full_weights", "vulkan_ctx",
                      "cuda_ctx", "act_cache", "current_frame_idx", "snapshot_writer", "train_tokens",
                      "num_samples", "current_epoch", "current_step", "current_loss", "nan_detected",
                      "optimizer_step", "accumulation_counter", "gradient_accumulation_steps", "learning_rate",
                      "debug", "debug_nan_check", "metrics_count", "vap_total_tracks"],
    "tensor_metadata_t": ["name", "dtype", "shape", "n_dims", "offset_start", "offset_end", "num_elements"],
    "safetensors_t": ["fd", "data", "file_size", "data_offset", "tensors", "num_tensors"],
    "tensor_location_t": ["name", "orig_name", "file_idx"],
    "seraph_model_t": ["st", "num_files", "tensor_map", "num_tensors", "config", "kv_cache", "lora", "act_cache"],
    "profiler_op_t": ["name", "event_start", "event_end", "elapsed_ms", "grid_x", "block_z", "shared_mem", "flops", "bytes"],
    "struct cuda_profiler_t": ["enabled", "num_ops", "ops", "total_step_ms", "total_other_ms", "log_file"],
}


def probe(includes, incdirs, tmp, tag):
    src = os.path.join(tmp, f"probe_{tag}.c")
    with open(src, "w") as f:
        f.write("#include <stdio.h>\n#include <stddef.h>\n")
        for inc in includes:
            f.write(f'#include "{inc}"\n')
        f.write("int main(void){\n")
        for st, fields in FIELDS.items():
            f.write(f'printf("{st} %zu\\n", sizeof({st}));\n')
            for fl in fields:
                f.write(f'printf("{st}.{fl} %zu\\n", offsetof({st}, {fl}));\n')
        f.write("return 0;}\n")
    exe = os.path.join(tmp, f"probe_{tag}")
    cmd = ["gcc", "-w", "-o", exe, src] + [f"-I{d}" for d in incdirs]
    subprocess.run(cmd, check=True)
    return subprocess.run([exe], check=True, capture_output=True, text=True).stdout


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "include")), reason="reference checkout not present")
def test_struct_layouts_match_reference():
    with tempfile.TemporaryDirectory() as tmp:
        ours = probe(["seraph_b200_abi.h"], [os.path.join(ROOT, "include")], tmp, "ours")
        theirs = probe(["train.h", "cuda_train_context.h", "cuda_profiler.h"], [os.path.join(REF, "include")], tmp, "ref")
    assert ours == theirs
