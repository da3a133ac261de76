"""Independent numpy (float64) implementations used to cross-check the C oracle on small shapes."""
import numpy as np


def dequant(packed, scales, k, n, group):
    packed = np.asarray(packed, dtype=np.uint32).reshape(k // 8, n)
    scales = np.asarray(scales, dtype=np.float32).reshape(-1, n)
    w = np.zeros((k, n), dtype=np.float32)
    for ki in range(k):
        nib = (packed[ki // 8] >> np.uint32(4 * (ki % 8))) & np.uint32(0xF)
        w[ki] = (nib.astype(np.int32) - 8).astype(np.float32) * scales[ki // group]
    return w


def quantize_weight_int4(w, k, n, group):
    w = np.asarray(w, dtype=np.float32).reshape(k, n)
    ng = (k + group - 1) // group
    scales = np.zeros((ng, n), dtype=np.float32)
    packed = np.zeros((k // 8, n), dtype=np.uint32)
    for g in range(ng):
        blk = w[g * group:(g + 1) * group]
        mx = np.abs(blk).max(axis=0).astype(np.float32)
        scales[g] = np.where(mx < np.float32(1e-12), np.float32(1.0), mx / np.float32(7.0))
    for ki in range(k):
        inv = np.float32(1.0) / scales[ki // group]
        v = w[ki] * inv
        q = np.clip(np.trunc(v + np.copysign(np.float32(0.5), v)).astype(np.int32), -8, 7)  # half away from zero
        packed[ki // 8] |= ((q + 8).astype(np.uint32) & np.uint32(0xF)) << np.uint32(4 * (ki % 8))
    return packed, scales


def layer_norm(x, g, b, eps):
    x = np.asarray(x, dtype=np.float64)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(g, np.float64) + np.asarray(b, np.float64)


def gelu_tanh(x):
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def gelu_sigmoid(x):
    x = np.asarray(x, dtype=np.float64)
    return x / (1.0 + np.exp(-1.702 * x))


def f16(x):
    return np.asarray(x, dtype=np.float64).astype(np.float16).astype(np.float64)


def gpt2_forward(cfg, w, tokens, gelu="tanh", kv_fp16=False, lm_head=None):
    """Full causal forward, float64, logits [seq, vocab]."""
    d, H = cfg["n_embd"], cfg["n_head"]
    dh = d // H
    t = np.asarray(tokens, dtype=np.int64)
    n = t.size
    h = w["wte"][t].astype(np.float64) + w["wpe"][:n].astype(np.float64)
    act = gelu_tanh if gelu == "tanh" else gelu_sigmoid
    mask = np.triu(np.ones((n, n), dtype=bool), 1)
    for i in range(cfg["n_layer"]):
        p = f"h.{i}."
        a = layer_norm(h, w[p + "ln_1.weight"], w[p + "ln_1.bias"], cfg.get("layer_norm_epsilon", 1e-5))
        qkv = a @ w[p + "attn.c_attn.weight"].astype(np.float64) + w[p + "attn.c_attn.bias"]
        q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
        if kv_fp16:
            k, v = f16(k), f16(v)
        out = np.zeros((n, d))
        for hd in range(H):
            sl = slice(hd * dh, (hd + 1) * dh)
            s = q[:, sl] @ k[:, sl].T / np.sqrt(dh)
            s[mask] = -np.inf
            s = np.exp(s - s.max(-1, keepdims=True))
            s /= s.sum(-1, keepdims=True)
            out[:, sl] = s @ v[:, sl]
        h = h + out @ w[p + "attn.c_proj.weight"].astype(np.float64) + w[p + "attn.c_proj.bias"]
        a = layer_norm(h, w[p + "ln_2.weight"], w[p + "ln_2.bias"], cfg.get("layer_norm_epsilon", 1e-5))
        f = act(a @ w[p + "mlp.c_fc.weight"].astype(np.float64) + w[p + "mlp.c_fc.bias"])
        h = h + f @ w[p + "mlp.c_proj.weight"].astype(np.float64) + w[p + "mlp.c_proj.bias"]
    hf = layer_norm(h, w["ln_f.weight"], w["ln_f.bias"], cfg.get("layer_norm_epsilon", 1e-5))
    if lm_head is not None:
        return hf @ np.asarray(lm_head, dtype=np.float64)
    return hf @ w["wte"].astype(np.float64).T


def rel_rms(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.sqrt(((a - b) ** 2).mean()) / (np.sqrt((b ** 2).mean()) + 1e-30))
