"""A plain, slow StarCoder2 written from the reference's formulas: whole sequences, no
cache, one function per part. It shares no code with ``matricxon_b200``: it has its own
reading of config keys, its own safetensors reader and its own sampler, so a mistake in
the engine cannot hide in a shared helper.

Each function cites the file and lines of nesmind/matricxon it restates. The comparison
with the reference's own model code on a tiny random model is tests/golden/ (script and
outputs); this file itself rests on the formulas.

All functions take and return CPU tensors. ``dtype`` is the arithmetic precision
(float64 for an oracle, float32 to mirror the reference bit for bit where possible);
rotary angles are always formed in float32, as the reference forms them.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------- configuration
def plain_config(raw: dict) -> dict:
    """Hyper-parameters as the reference derives them (app/architectures/starcoder2.py:63-79):
    KV heads default to the head count (:67), head_dim to hidden // heads (:68)."""
    heads = raw["num_attention_heads"]
    window = raw.get("sliding_window")
    return {
        "hidden": raw["hidden_size"],
        "layers": raw["num_hidden_layers"],
        "heads": heads,
        "kv_heads": raw.get("num_key_value_heads") or heads,
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
        "intermediate": raw["intermediate_size"],
        "vocab": raw["vocab_size"],
        "theta": float(raw["rope_theta"]),
        "window": window if window else None,
        "eps": float(raw["norm_epsilon"]),
        "bias": raw.get("use_bias", True),
        "tied": raw.get("tie_word_embeddings", True),
    }


# --------------------------------------------------------------------------- weights
_ST_DTYPES = {"F32": (np.float32, torch.float32), "BF16": (np.uint16, torch.bfloat16),
              "F16": (np.float16, torch.float16), "I32": (np.int32, torch.int32),
              "I64": (np.int64, torch.int64)}


def plain_read_safetensors(path: str | Path) -> dict[str, torch.Tensor]:
    """name -> float32 tensor (integers stay integers)."""
    data = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + length])
    body = data[8 + length:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_dtype, torch_dtype = _ST_DTYPES[info["dtype"]]
        begin, end = info["data_offsets"]
        array = np.frombuffer(body[begin:end], dtype=np_dtype).copy().reshape(info["shape"])
        tensor = torch.from_numpy(array)
        if torch_dtype == torch.bfloat16:
            tensor = tensor.view(torch.bfloat16)
        out[name] = tensor.float() if tensor.is_floating_point() else tensor
    return out


def plain_load_model(folder: str | Path) -> tuple[dict, dict[str, torch.Tensor]]:
    folder = Path(folder)
    raw = json.loads((folder / "config.json").read_text())
    return plain_config(raw), plain_read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------- parts
def plain_embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x = E[ids] (app/architectures/starcoder2.py:218)."""
    return table[ids]


def plain_layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                    eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight + bias, biased variance over the last axis:
    nn.LayerNorm as used at app/architectures/starcoder2_layers.py:45,56 and
    app/architectures/starcoder2.py:97."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mean) / torch.sqrt(var + eps) * weight
    return y + bias if bias is not None else y


def plain_rope_tables(positions: torch.Tensor, dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq = 1 / theta^(arange(0, dim, 2)/dim); freqs = pos.float() * inv_freq;
    emb = cat(freqs, freqs); cos, sin -- all float32 (app/architectures/rope.py:16-29)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = positions.float().unsqueeze(-1) * inv_freq
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def plain_rotate_half(x: torch.Tensor) -> torch.Tensor:
    """[-x2, x1] with x1, x2 the two halves of the last axis (app/architectures/rope.py:152-154)."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([-x2, x1], dim=-1)


def plain_apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x * cos + rotate_half(x) * sin; x is [heads, T, dim], tables [T, dim]
    (app/architectures/rope.py:157-169)."""
    cos, sin = cos.to(x.dtype).unsqueeze(0), sin.to(x.dtype).unsqueeze(0)
    return x * cos + plain_rotate_half(x) * sin


def plain_mask(q_len: int, kv_len: int, offset: int, window: int | None) -> torch.Tensor:
    """Query i (absolute position i + offset) sees key j iff j <= i + offset
    (app/architectures/qwen_layers.py:12-17) and, with a window, j > i + offset - window
    (app/architectures/gemma4_layers.py:17-34; app/native/src/mx_attention.c:36-39)."""
    q_idx = torch.arange(q_len).unsqueeze(1) + offset
    kv_idx = torch.arange(kv_len).unsqueeze(0)
    mask = kv_idx <= q_idx
    if window is not None:
        mask = mask & (kv_idx > q_idx - window)
    return mask


def plain_attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                         window: int | None, offset: int = 0) -> torch.Tensor:
    """q [heads, Tq, d], k and v [kv_heads, Tk, d] -> [heads, Tq, d]. Scores q.k * scale,
    max-subtracted softmax over visible keys, weighted sum of values; query head h reads KV
    head h // (heads / kv_heads) (app/native/src/mx_attention.c:16-68;
    app/architectures/qwen_layers.py:94-100)."""
    heads, q_len, _ = q.shape
    group = heads // k.shape[0]
    mask = plain_mask(q_len, k.shape[1], offset, window)
    out = torch.empty_like(q)
    for h in range(heads):
        kh, vh = k[h // group], v[h // group]
        scores = (q[h] @ kh.T) * scale
        scores = scores.masked_fill(~mask, float("-inf"))
        scores = scores - scores.max(dim=-1, keepdim=True).values
        weights = torch.exp(scores)
        weights = weights / weights.sum(dim=-1, keepdim=True)
        out[h] = weights @ vh
    return out


def plain_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """x W^T + b with W stored (out, in) (nn.Linear, app/architectures/qwen_layers.py:50-53)."""
    y = x @ weight.T
    return y + bias if bias is not None else y


def plain_attention(h: torch.Tensor, w: dict, prefix: str, cfg: dict,
                    positions: torch.Tensor) -> torch.Tensor:
    """Projections, head split (feature head * d + i), RoPE on q and k, attention, output
    projection (app/architectures/qwen_layers.py:69-102)."""
    t = h.shape[0]
    heads, kv_heads, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]

    def proj(name):
        return plain_linear(h, w[f"{prefix}{name}.weight"],
                            w.get(f"{prefix}{name}.bias") if cfg["bias"] else None)

    q = proj("q_proj").view(t, heads, d).transpose(0, 1)
    k = proj("k_proj").view(t, kv_heads, d).transpose(0, 1)
    v = proj("v_proj").view(t, kv_heads, d).transpose(0, 1)
    cos, sin = plain_rope_tables(positions, d, cfg["theta"])
    q, k = plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin)
    o = plain_attention_core(q, k, v, d ** -0.5, cfg["window"])
    o = o.transpose(0, 1).reshape(t, heads * d)
    return plain_linear(o, w[f"{prefix}o_proj.weight"],
                        w.get(f"{prefix}o_proj.bias") if cfg["bias"] else None)


def plain_gelu_tanh(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3))): F.gelu(approximate="tanh") at
    app/architectures/starcoder2_layers.py:23."""
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u ** 3)))


def plain_mlp(h: torch.Tensor, w: dict, prefix: str, cfg: dict) -> torch.Tensor:
    """down(gelu_tanh(up(h))) (app/architectures/starcoder2_layers.py:9-23)."""
    up = plain_linear(h, w[f"{prefix}c_fc.weight"], w.get(f"{prefix}c_fc.bias") if cfg["bias"] else None)
    return plain_linear(plain_gelu_tanh(up), w[f"{prefix}c_proj.weight"],
                        w.get(f"{prefix}c_proj.bias") if cfg["bias"] else None)


def plain_layer(x: torch.Tensor, w: dict, index: int, cfg: dict, positions: torch.Tensor) -> torch.Tensor:
    """x = x + attn(LN1(x)); x = x + mlp(LN2(x)) (app/architectures/starcoder2_layers.py:67-68)."""
    p = f"model.layers.{index}."
    h = plain_layernorm(x, w[p + "input_layernorm.weight"], w[p + "input_layernorm.bias"], cfg["eps"])
    x = x + plain_attention(h, w, p + "self_attn.", cfg, positions)
    h = plain_layernorm(x, w[p + "post_attention_layernorm.weight"],
                        w[p + "post_attention_layernorm.bias"], cfg["eps"])
    return x + plain_mlp(h, w, p + "mlp.", cfg)


def plain_forward(cfg: dict, weights: dict[str, torch.Tensor], ids: list[int] | torch.Tensor,
                  dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (app/architectures/starcoder2.py:204-233)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    positions = torch.arange(ids.shape[0])
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    for index in range(cfg["layers"]):
        x = plain_layer(x, w, index, cfg, positions)
    x = plain_layernorm(x, w["model.norm.weight"], w["model.norm.bias"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return x @ head.T


# --------------------------------------------------------------------------- sampling
def plain_repeat_penalty(logits: torch.Tensor, generated: list[int], penalty: float) -> torch.Tensor:
    """Positive scores of already generated ids are divided by the penalty, negative ones
    multiplied (app/runtime/sampler.py:12-26)."""
    if penalty == 1.0 or not generated:
        return logits
    logits = logits.clone()
    for token in set(generated):
        logits[token] = logits[token] / penalty if logits[token] > 0 else logits[token] * penalty
    return logits


def plain_top_k(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Keeps every logit >= the k-th largest, ties included (app/runtime/sampler.py:44-52)."""
    if k <= 0 or k >= logits.shape[-1]:
        return logits
    threshold = torch.topk(logits, k).values[-1]
    return logits.masked_fill(logits < threshold, float("-inf"))


def plain_top_p(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Keeps a token iff the probability mass of the tokens ranked before it is <= p; always
    the best one (app/runtime/sampler.py:55-73; app/native/src/mx_sample.c:88-99)."""
    if p >= 1.0:
        return logits
    sorted_logits, order = torch.sort(logits, descending=True)
    probs = torch.softmax(sorted_logits.double(), dim=-1)
    before = torch.cumsum(probs, dim=-1) - probs
    sorted_logits = sorted_logits.masked_fill(before > p, float("-inf"))
    out = torch.full_like(logits, float("-inf"))
    out[order] = sorted_logits
    return out


def plain_draw(logits: torch.Tensor, u: float) -> int:
    """Inverse CDF in vocabulary order: exp(x - max) summed in double, the first index whose
    running sum exceeds u * total (app/native/src/mx_sample.c:82-107)."""
    keep = torch.isfinite(logits)
    peak = logits[keep].max()
    weights = torch.where(keep, torch.exp((logits - peak).float()).double(), torch.zeros((), dtype=torch.float64))
    running = torch.cumsum(weights, dim=0)
    target = u * running[-1]
    hits = torch.nonzero(running > target)
    if hits.numel() == 0:
        return int(torch.nonzero(keep)[-1])
    return int(hits[0])


def plain_sample(logits: torch.Tensor, generated: list[int], temperature: float, top_k: int,
                 top_p: float, repeat_penalty: float, u: float) -> int:
    """repeat penalty -> (temperature <= 0: argmax) -> / temperature -> top-k -> top-p -> draw
    (app/runtime/sampler.py:93-129)."""
    logits = plain_repeat_penalty(logits.float(), generated, repeat_penalty)
    if temperature <= 0.0:
        return int(torch.argmax(logits))
    logits = logits / temperature
    logits = plain_top_k(logits, top_k)
    logits = plain_top_p(logits, top_p)
    return plain_draw(logits, u)
