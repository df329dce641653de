"""Plain, slow Qwen3-dense forward for whole sequences: no cache, no batching, no kernels.

Written from the formulas of the reference's CPU backend (file:line cited per function, paths
within the reference project).  It shares no code with ``ember_b200``: it parses config.json
and the safetensors file itself and computes with torch on the CPU, in float64 by default
(the reference uses float32 with float64 for two reductions; float64 throughout is the
stricter oracle) or float32.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# --------------------------------------------------------------------------- model files
def read_config(model_dir: str) -> dict:
    """Keys and defaults as src/model/config.cpp:18-42."""
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    return {
        "vocab": c["vocab_size"], "hidden": c["hidden_size"], "inter": c["intermediate_size"],
        "layers": c["num_hidden_layers"], "heads": heads,
        "kv_heads": c.get("num_key_value_heads") or heads,
        "head_dim": c.get("head_dim") or c["hidden_size"] // heads,
        "eps": c.get("rms_norm_eps", 1e-6) if c.get("rms_norm_eps") is not None else 1e-6,
        "theta": c.get("rope_theta", 10000.0) if c.get("rope_theta") is not None else 10000.0,
        "tie": bool(c.get("tie_word_embeddings", False)),
        "bias": bool(c.get("attention_bias", False)),
        # not in the reference (it ignores these keys): the layers from max_window_layers on see only the last
        # sliding_window keys, their own position included
        "window": int(c.get("sliding_window") or 0) if c.get("use_sliding_window") else 0,
        "window_from": int(c.get("max_window_layers") or 0),
    }


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw data (src/model/safetensors.cpp:54-82)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    data = blob[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        dt = info["dtype"]
        if dt == "F32":
            t = torch.from_numpy(raw.view(np.float32).copy())
        elif dt == "BF16":
            # bfloat16 is the upper half of a float32
            u = raw.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif dt == "F16":
            t = torch.from_numpy(raw.view(np.float16).astype(np.float32))
        else:
            raise ValueError(f"unsupported dtype {dt}")
        out[name] = t.reshape(info["shape"])
    return out


# ------------------------------------------------------------------------------- parts
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """out_i = w_i * (x_i * 1/sqrt(mean(x^2) + eps)) over the last axis (cpu_backend.cpp:34-39)."""
    ss = (x.double() * x.double()).sum(-1, keepdim=True)
    scale = (1.0 / torch.sqrt(ss / x.shape[-1] + eps)).to(x.dtype)
    return w * (x * scale)


def embedding(table: torch.Tensor, tokens: List[int]) -> torch.Tensor:
    """h[t] = table[token[t]], no scaling (cpu_backend.cpp:131-135)."""
    return table[torch.tensor(tokens, dtype=torch.long)]


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x . W^T (+ b) with W [out, in] (src/backend/cpu/cpu_kernels.hpp:25)."""
    y = x @ w.t()
    return y + b if b is not None else y


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq_i = 1 / powf(float(theta), float(2i) / float(D)) in float32 (cpu_backend.cpp:85-88)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    e = (np.float32(2.0) * i) / np.float32(head_dim)
    return torch.from_numpy((np.float32(1.0) / np.power(np.float32(theta), e, dtype=np.float32)).astype(np.float32))


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half: pairs (x_i, x_{i+D/2}); angle = float(pos) * inv_freq_i in float32
    (cpu_backend.cpp:263-272).  x: [T, heads, D]."""
    half = x.shape[-1] // 2
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # float32 product
    cs, sn = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0,
              scale: Optional[float] = None) -> torch.Tensor:
    """Causal grouped-query attention of a whole sequence (cpu_backend.cpp:138, 174-198):
    s_j = dot(q_h, k_{h / group, j}) * 1/sqrt(D) for j <= t (and j > t - window if a window is
    given), softmax over j, o = sum_j w_j v_j.   q: [T, heads, D]; k, v: [T, kv_heads, D]."""
    T, H, D = q.shape
    group = H // k.shape[1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.zeros_like(q)
    for h in range(H):
        kh, vh = k[:, h // group], v[:, h // group]
        s = (q[:, h] @ kh.t()) * scale                                        # [T, T]
        t = torch.arange(T)
        visible = t[None, :] <= t[:, None]
        if window > 0:
            visible &= t[None, :] > t[:, None] - window
        s = s.masked_fill(~visible, float("-inf"))
        w = torch.softmax(s, dim=-1)
        out[:, h] = w @ vh
    return out


def swiglu(x: torch.Tensor, gate_w, up_w, down_w) -> torch.Tensor:
    """down( g / (1 + exp(-g)) * u ) with g = x.Wg^T, u = x.Wu^T (cpu_backend.cpp:204-211)."""
    g, u = linear(x, gate_w), linear(x, up_w)
    return linear(g / (1.0 + torch.exp(-g)) * u, down_w)


def attention_block(x, w: Dict[str, torch.Tensor], p: str, cfg: dict, positions, inv_freq, window: int = 0):
    """q/k/v projections (+bias), per-head q/k RMSNorm with the layer eps, rotation, attention,
    output projection (cpu_backend.cpp:143-200)."""
    T = x.shape[0]
    H, KV, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    bias = (lambda n: w[p + n + ".bias"]) if cfg["bias"] else (lambda n: None)
    q = linear(x, w[p + "q_proj.weight"], bias("q_proj")).view(T, H, D)
    k = linear(x, w[p + "k_proj.weight"], bias("k_proj")).view(T, KV, D)
    v = linear(x, w[p + "v_proj.weight"], bias("v_proj")).view(T, KV, D)
    q = rope(rmsnorm(q, w[p + "q_norm.weight"], cfg["eps"]), positions, inv_freq)
    k = rope(rmsnorm(k, w[p + "k_norm.weight"], cfg["eps"]), positions, inv_freq)
    o = attention(q, k, v, window=window).reshape(T, H * D)
    return linear(o, w[p + "o_proj.weight"])


# ------------------------------------------------------------------------------- model
class PlainQwen3:
    def __init__(self, model_dir: str, dtype: torch.dtype = torch.float64):
        self.cfg = read_config(model_dir)
        raw = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        self.w = {n: t.to(dtype) for n, t in raw.items()}
        self.dtype = dtype
        self.inv_freq = rope_inv_freq(self.cfg["head_dim"], self.cfg["theta"])

    def hidden_states(self, tokens: List[int]) -> List[torch.Tensor]:
        """Residual stream after the embedding and after every layer, [T, hidden] each
        (pre-norm decoder, cpu_backend.cpp:139-213)."""
        c, w = self.cfg, self.w
        pos = torch.arange(len(tokens))
        h = embedding(w["model.embed_tokens.weight"], tokens)
        out = [h]
        for l in range(c["layers"]):
            p = f"model.layers.{l}."
            x = rmsnorm(h, w[p + "input_layernorm.weight"], c["eps"])
            window = c["window"] if l >= c["window_from"] else 0
            h = h + attention_block(x, w, p + "self_attn.", c, pos, self.inv_freq, window=window)
            x = rmsnorm(h, w[p + "post_attention_layernorm.weight"], c["eps"])
            h = h + swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
            out.append(h)
        return out

    def logits(self, tokens: List[int]) -> torch.Tensor:
        """Logits at every position, [T, vocab] float32: final norm, then the head; the head is
        the embedding when tied or when lm_head.weight is absent (cpu_backend.cpp:51-53, 215-224)."""
        c, w = self.cfg, self.w
        h = self.hidden_states(tokens)[-1]
        n = rmsnorm(h, w["model.norm.weight"], c["eps"])
        head = w["model.embed_tokens.weight"] if c["tie"] or "lm_head.weight" not in w else w["lm_head.weight"]
        return linear(n, head).to(torch.float32)

    def greedy(self, prompt: List[int], n: int) -> List[int]:
        """n greedy tokens, recomputing the whole sequence each time; ties go to the lowest id
        (src/backend/sampling_host.cpp:22-28)."""
        toks = list(prompt)
        out = []
        for _ in range(n):
            row = self.logits(toks)[-1]
            best = int(torch.argmax(row))          # torch returns the first maximum
            out.append(best)
            toks.append(best)
        return out
