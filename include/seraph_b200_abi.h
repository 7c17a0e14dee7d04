/*
 * seraph_b200_abi.h - the data contract of Seraph's C training API, restated.
 *
 * libseraph_b200 is called by programs that were compiled against Seraph's own
 * headers, so the layouts below must stay byte-compatible with:
 *   cuda_buffer_t, cuda_lora_gpu_*_t, cuda_train_context_t  include/cuda_train_context.h:15-233
 *   weight_tensor_t, layer_weights_t, trainable_weights_t     include/train.h:53-90
 *   train_state_t                                             include/train.h:183-320
 *   model_config_t                                            include/model_config.h:34-106
 *   lora_adapter_t, lora_model_t                              include/lora.h:13-56
 *   profiler_op_t, cuda_profiler_t                            include/cuda_profiler.h:21-50
 * Fields this library never touches are folded into arrays of the same size
 * and alignment.  tests/test_abi_layout.py compiles both sets of headers and
 * compares sizeof/offsetof for every field used.
 */
#ifndef SERAPH_B200_ABI_H
#define SERAPH_B200_ABI_H

#include <stddef.h>
#include <stdint.h>
#include <stdbool.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device buffers -------------------------------------------------- */
typedef struct { float* data; size_t size; } cuda_buffer_t;   /* size in bytes */

typedef struct {
    cuda_buffer_t **A, **B, **gA, **gB, **mA, **vA, **mB, **vB;   /* each [num_layers], NULL entries allowed */
    int active;
} cuda_lora_gpu_adapter_t;

typedef struct {
    int num_layers, rank;
    float alpha, scale;                                          /* scale = alpha / rank */
    cuda_lora_gpu_adapter_t q, k, v, o, gate, up, down;
} cuda_lora_gpu_state_t;

/* ---- the context: every field is ABI (callers read and write some directly,
 *      tools/seraph_train_cuda.c:216-264, :455) ---------------------------- */
typedef struct {
    int device_id;
    void* stream;                       /* cudaStream_t */
    int initialized;
    int gpu_sm_count, gpu_max_threads_per_block, gpu_shared_mem_per_block, gpu_shared_mem_per_sm,
        gpu_warp_size, gpu_compute_major, gpu_compute_minor, gpu_l2_cache_bytes,
        gpu_max_shared_per_block_optin, gpu_max_threads_per_sm, gpu_regs_per_sm;
    int use_bf16;                       /* 1: BF16 tensor-core GEMM mode */
    int use_flash_attn;                 /* accepted; attention here is always tiled and keeps the LSE */
    int batch_size;
    int matmul_tile_dim, matmul_block_k, parallel_block_size, attention_block_size, attention_num_warps;

    cuda_buffer_t *weight_buffer, *grad_buffer, *m_buffer, *v_buffer;
    size_t max_buffer_size;
    cuda_buffer_t *fwd_input_buffer, *fwd_weight_buffer, *fwd_output_buffer;
    size_t max_fwd_buffer_size;
    cuda_buffer_t *attn_q_buffer, *attn_k_buffer, *attn_v_buffer, *attn_out_buffer;
    size_t max_attn_buffer_size;
    cuda_buffer_t *fwd_hidden_buffer, *fwd_hidden_norm_buffer, *fwd_tmp_hidden_buffer, *fwd_ffn_gate_buffer,
                  *fwd_ffn_up_buffer, *fwd_ffn_hidden_buffer, *fwd_logits_buffer, *fwd_norm_weight_buffer;
    size_t max_fwd_act_bytes;

    int fwd_cache_num_layers, fwd_cache_max_seq, fwd_cache_hidden_size, fwd_cache_intermediate_size, fwd_cache_q_dim;
    cuda_buffer_t **fwd_cache_x_norm_attn, **fwd_cache_x_norm_ffn, **fwd_cache_attn_out, **fwd_cache_ffn_gate_out,
                  **fwd_cache_ffn_up_out, **fwd_cache_ffn_hidden, **fwd_cache_layer_input, **fwd_cache_post_attn_in,
                  **fwd_cache_silu_out, **fwd_cache_q, **fwd_cache_k, **fwd_cache_v, **fwd_cache_attn_lse;

    cuda_buffer_t *train_tokens_u32, *train_targets_u32, *train_grad_logits, *train_loss_rows,
                  *train_reduce_tmp_a, *train_reduce_tmp_b, *train_seq_starts, *train_grad_hidden,
                  *train_grad_tmp_hidden, *train_grad_x_norm, *train_grad_q, *train_grad_k, *train_grad_v,
                  *train_grad_attn, *train_grad_ffn, *train_grad_gate, *train_grad_up, *train_final_input;

    int gpu_weights_num_layers, gpu_weights_hidden_size, gpu_weights_intermediate_size,
        gpu_weights_q_dim, gpu_weights_kv_dim, gpu_weights_vocab_size;

    cuda_buffer_t *gpu_w_embed, *gpu_g_embed, *gpu_m_embed, *gpu_v_embed;
    cuda_buffer_t *gpu_w_final_norm, *gpu_g_final_norm, *gpu_m_final_norm, *gpu_v_final_norm;
    /* per-layer arrays [num_layers]: weight, gradient, Adam m, Adam v */
    cuda_buffer_t **gpu_w_q, **gpu_g_q, **gpu_m_q, **gpu_v_q;
    cuda_buffer_t **gpu_w_k, **gpu_g_k, **gpu_m_k, **gpu_v_k;
    cuda_buffer_t **gpu_w_v, **gpu_g_v, **gpu_m_v, **gpu_v_v;
    cuda_buffer_t **gpu_w_o, **gpu_g_o, **gpu_m_o, **gpu_v_o;
    cuda_buffer_t **gpu_w_gate, **gpu_g_gate, **gpu_m_gate, **gpu_v_gate;
    cuda_buffer_t **gpu_w_up, **gpu_g_up, **gpu_m_up, **gpu_v_up;
    cuda_buffer_t **gpu_w_down, **gpu_g_down, **gpu_m_down, **gpu_v_down;
    cuda_buffer_t **gpu_w_in_norm, **gpu_g_in_norm, **gpu_m_in_norm, **gpu_v_in_norm;
    cuda_buffer_t **gpu_w_post_norm, **gpu_g_post_norm, **gpu_m_post_norm, **gpu_v_post_norm;

    cuda_buffer_t* debug_nan_flags;
    void* lora_gpu;                     /* cuda_lora_gpu_state_t* */
    cuda_buffer_t* lora_hidden_tmp;
    size_t lora_hidden_tmp_bytes;
} cuda_train_context_t;

/* ---- host-side model / training state -------------------------------- */
typedef struct { float *weight, *grad, *m, *v; size_t size; } weight_tensor_t;

typedef struct {
    weight_tensor_t q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj, input_norm, post_norm;
} layer_weights_t;

typedef struct {
    int num_layers, hidden_size, intermediate_size, vocab_size;
    layer_weights_t* layers;
    weight_tensor_t embed_tokens, final_norm;
    size_t total_params;
} trainable_weights_t;

typedef struct {
    int in_dim, out_dim, rank;
    float alpha;
    float *A, *B, *grad_A, *grad_B, *m_A, *v_A, *m_B, *v_B;   /* A [rank,in], B [out,rank] */
} lora_adapter_t;

typedef struct {
    int num_layers, rank;
    float alpha, dropout;
    int apply_to_q, apply_to_k, apply_to_v, apply_to_o, apply_to_ffn;
    lora_adapter_t **q_adapters, **k_adapters, **v_adapters, **o_adapters,
                   **gate_adapters, **up_adapters, **down_adapters;
} lora_model_t;

typedef struct {
    char model_name[256];
    char model_type[64];
    int arch;                            /* model_arch_t */
    int vocab_size, hidden_size, num_hidden_layers, intermediate_size;
    int num_attention_heads, num_key_value_heads, head_dim, kv_dim;
    float rms_norm_eps;                  /* ignored by training: eps is 1e-5 (src/train_cuda.c:1984) */
    float rope_theta;
    int max_position_embeddings;
    int use_qk_norm;
    int video_ints_[15];                 /* patch_size[3] .. mask_dim, clip_embed_dim */
    char clip_embeddings_path[512];
    float clip_loss_weight;
    char hidden_act[32];
    int bos_token_id, eos_token_id, pad_token_id;
    int chat_format;                     /* chat_format_t */
    char chat_tokens_[32 + 32 + 64 + 64 + 64];
    bool tie_word_embeddings;
    char torch_dtype[16];
    int num_model_files;
    char model_dir[512];
} model_config_t;

/* ---- the model the frozen LoRA base is read from: include/safetensors.h:25-45, include/transformer.h:15-43 -------- */
typedef struct {
    char* name;
    int dtype;                           /* dtype_t: 1 F32, 2 F16, 3 BF16 */
    int64_t* shape;
    int n_dims;
    int64_t offset_start, offset_end;    /* bytes from the start of the data section */
    size_t num_elements;
} tensor_metadata_t;

typedef struct {
    int fd;
    uint8_t* data;                       /* the whole file, memory-mapped */
    size_t file_size, data_offset;       /* data_offset = 8 + header length */
    tensor_metadata_t* tensors;
    int num_tensors;
} safetensors_t;

typedef struct { char name[256]; char orig_name[256]; int file_idx; } tensor_location_t;

typedef struct {
    safetensors_t* st[8];
    int num_files;
    tensor_location_t* tensor_map;
    int num_tensors;
    model_config_t* config;
    void* kv_cache;
    lora_model_t* lora;
    void* act_cache;
} seraph_model_t;

typedef struct {
    void *model;                         /* seraph_model_t* */
    model_config_t* config;
    void *tokenizer, *train_cfg;
    int use_full_training;
    lora_model_t* lora;
    trainable_weights_t* full_weights;
    void *vulkan_ctx, *cuda_ctx;
    size_t max_tensor_size;
    void* act_cache;
    void* video_state_[12];
    int current_frame_idx, valid_query_count;
    void* video_heads_[9 + 12 + 9];
    void* snapshot_writer;
    int* train_tokens; int num_train_tokens;
    int* sample_offsets; int num_samples;
    float* video_frames; int* video_labels; float* video_masks;
    int num_video_frames, num_labels_per_frame;
    void* vdat_mmap; size_t vdat_mmap_size;
    void *gpu_mask_targets, *gpu_mask_loss, *gpu_grad_mask;
    float* val_video_frames; int* val_video_labels; float* val_video_masks;
    int num_val_video_frames;
    int current_epoch, current_step, total_steps;
    float current_loss, best_val_loss;
    int nan_detected;
    int optimizer_step, accumulation_counter, gradient_accumulation_steps;
    float learning_rate;
    int debug, debug_weight_delta, debug_nan_check;
    float vision_metrics_[10];
    int metrics_count;
    int* prev_query_classes; float* prev_query_conf;
    int vap_id_switches, vap_total_tracks;
} train_state_t;

/* ---- profiler -------------------------------------------------------- */
#define PROFILER_MAX_OPS 1024
typedef struct {
    char name[80];
    void *event_start, *event_end;       /* cudaEvent_t */
    float elapsed_ms;
    int grid_x, grid_y, grid_z, block_x, block_y, block_z;
    size_t shared_mem, flops, bytes;
} profiler_op_t;

typedef struct cuda_profiler_t {
    int enabled, num_ops;
    profiler_op_t ops[PROFILER_MAX_OPS];
    float total_step_ms, total_matmul_ms, total_attention_ms, total_attention_bwd_ms, total_rmsnorm_ms,
          total_rmsnorm_bwd_ms, total_cross_entropy_ms, total_adamw_ms, total_copy_ms, total_other_ms;
    void* log_file;                      /* FILE* */
} cuda_profiler_t;

#ifdef __cplusplus
}
#endif
#endif
