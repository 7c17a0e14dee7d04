"""float64 torch restatement of the decoder the reference trains, used only to
cross-check the C oracle's chain rule with autograd (and as the oracle for
shapes too large for the C loops, on a GPU).  Same conventions as the
reference: interleaved-pair RoPE, kv head = h*Hkv//Hq, RMSNorm eps 1e-5, tied
LM head, packed sequences with a causal mask per sequence, mean loss over the
T-B valid predictions (src/train_cuda.c:1966-2326)."""
import numpy as np
import torch


def unflatten(cfg, flat, device="cpu", dtype=torch.float64, requires_grad=True):
    out = {}
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        t = torch.tensor(flat[off:off + n].reshape(shp), dtype=dtype, device=device)
        t.requires_grad_(requires_grad)
        out[name] = t
    return out


def flatten_grads(cfg, P):
    g = np.zeros(cfg.n_params(), np.float64)
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        if P[name].grad is not None:
            g[off:off + n] = P[name].grad.detach().cpu().numpy().ravel()
    return g


def rope(x, pos, H, hd, theta):
    T = x.shape[0]
    x = x.view(T, H, hd // 2, 2)
    p = torch.arange(hd // 2, device=x.device, dtype=torch.float32)
    # angle built in fp32 exactly as the kernels do: pos * (1/powf(theta, 2p/hd))
    freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32, device=x.device), (p * 2) / hd)
    ang = (pos.to(torch.float32)[:, None] * freq[None, :]).to(x.dtype)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., 0], x[..., 1]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).reshape(T, H * hd)


def rmsnorm(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def unflatten_extras(cfg, flat, device="cpu", dtype=torch.float64, requires_grad=True):
    out = {}
    for name, shp, off in cfg.extras_tensors()[0]:
        n = int(np.prod(shp))
        out[name] = torch.tensor(flat[off:off + n].reshape(shp), dtype=dtype, device=device).requires_grad_(requires_grad)
    return out


def forward_loss(cfg, P, tokens, seq_starts, lora=None, rank=0, alpha=0.0, X=None):
    dev = P["embed"].device
    T, B = len(tokens), len(seq_starts) - 1
    tok = torch.tensor(np.maximum(np.asarray(tokens), 0), dtype=torch.long, device=dev)
    seq_id = torch.zeros(T, dtype=torch.long, device=dev)
    pos = torch.zeros(T, dtype=torch.long, device=dev)
    valid = torch.ones(T, dtype=torch.bool, device=dev)
    for b in range(B):
        s, e = seq_starts[b], seq_starts[b + 1]
        seq_id[s:e] = b
        pos[s:e] = torch.arange(e - s, device=dev)
        valid[e - 1] = False
    idx = torch.arange(T, device=dev)
    mask = (seq_id[:, None] == seq_id[None, :]) & (idx[None, :] <= idx[:, None])
    s_l = alpha / rank if rank else 0.0

    def lin(x, name):
        y = x @ P[name].T
        if lora is not None and name + ".A" in lora:
            y = y + (s_l * (x @ lora[name + ".A"].T)) @ lora[name + ".B"].T
        return y

    h = P["embed"][tok]
    g = cfg.Hq // cfg.Hkv
    for l in range(cfg.L):
        x = rmsnorm(h, P[f"l{l}.in_norm"], cfg.eps)
        q, k = lin(x, f"l{l}.q"), lin(x, f"l{l}.k")
        if getattr(cfg, "head_norm", 0) and X is not None:      # learned RMSNorm over each head, before RoPE
            q = rmsnorm(q.view(T, cfg.Hq, cfg.hd), X[f"l{l}.q_norm"], cfg.eps).reshape(T, cfg.qd)
            k = rmsnorm(k.view(T, cfg.Hkv, cfg.hd), X[f"l{l}.k_norm"], cfg.eps).reshape(T, cfg.kvd)
        q = rope(q, pos, cfg.Hq, cfg.hd, cfg.theta)
        k = rope(k, pos, cfg.Hkv, cfg.hd, cfg.theta)
        if getattr(cfg, "qk_norm", 0):           # whole-row normalisation after RoPE (shaders/qk_norm.comp)
            q = q.reshape(T, -1); k = k.reshape(T, -1)
            q = q / torch.clamp(torch.sqrt((q * q).mean(dim=1, keepdim=True)), min=cfg.eps)
            k = k / torch.clamp(torch.sqrt((k * k).mean(dim=1, keepdim=True)), min=cfg.eps)
        q = q.reshape(T, cfg.Hq, cfg.hd); k = k.reshape(T, cfg.Hkv, cfg.hd)
        v = lin(x, f"l{l}.v").view(T, cfg.Hkv, cfg.hd)
        kv_of = (torch.arange(cfg.Hq, device=dev) * cfg.Hkv) // cfg.Hq
        kk, vv = k[:, kv_of], v[:, kv_of]
        sc = torch.einsum("thd,shd->hts", q, kk) / np.sqrt(cfg.hd)
        sc = sc.masked_fill(~mask[None], float("-inf"))
        att = torch.einsum("hts,shd->thd", torch.softmax(sc, -1), vv).reshape(T, cfg.qd)
        h = h + lin(att, f"l{l}.o")
        x = rmsnorm(h, P[f"l{l}.post_norm"], cfg.eps)
        ff = torch.nn.functional.silu(lin(x, f"l{l}.gate")) * lin(x, f"l{l}.up")
        h = h + lin(ff, f"l{l}.down")
    head = X["lm_head"] if (getattr(cfg, "untied", 0) and X is not None) else P["embed"]
    logits = rmsnorm(h, P["final_norm"], cfg.eps) @ head.T
    tgt = torch.zeros(T, dtype=torch.long, device=dev)
    tgt[:-1] = tok[1:]
    lp = torch.log_softmax(logits, -1)
    nll = -lp[idx, tgt]
    loss = (nll * valid).sum() / (T - B)
    return loss, logits
