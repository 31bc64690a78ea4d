"""Plain, slow restatement of the Tekosun design in torch on the CPU — one function per mechanism, written from the
design's equations and sharing no code with the package.  It takes the config as the plain dict config.json holds and the
weights under their checkpoint names (as float tensors).

Tekosun: a residual stream x [T, width]; every layer is  x += rms_a(mixer(x))  then  x += rms_b(ff(x))  — the norm sits on
the sublayer's OUTPUT only, the sublayers read x itself.  Mixers: a generalized delta rule (per head a key × value matrix
state with a per-channel decay and a rank-one removal along the unit key), Mamba-2 (a short causal convolution and a
scalar-decay state-space recurrence per head), or a sliding-window softmax attention with whole-projection query / key
norms, rotate-half rotary positions on the first dims of each head with Llama-3.1 frequency scaling, unit-rms values and
a mix-in of the first such layer's values.  Feed-forwards are softmax-routed squared-ReLU experts with renormalised top
weights plus an always-on shared expert.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------------------- norms
def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(v, eps) * w


# -------------------------------------------------------------------------------------------------------------- rotary
def rotary_frequencies(rot: dict) -> torch.Tensor:
    """Angular frequency of every pair [dims/2] (float64), with the Llama-3.1 rescaling of long wavelengths."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, lo, hi, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    wave = 2.0 * math.pi / f
    s = (orig / wave - lo) / (hi - lo)
    mid = (1.0 - s) * f / factor + s * f
    return torch.where(wave < orig / hi, f, torch.where(wave > orig / lo, f / factor, mid))


def rotate_half(v: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """v [T, heads, n]: entry i of the first rot.dims entries is paired with entry i + dims/2."""
    dims = int(rot["dims"])
    h = dims // 2
    ang = positions.to(torch.float64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(ang).to(v.dtype)[:, None, :], torch.sin(ang).to(v.dtype)[:, None, :]
    a, b = v[..., :h], v[..., h:dims]
    out = v.clone()
    out[..., :h] = a * c - b * s
    out[..., h:dims] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------------------- attention
def attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float,
              v_first: Optional[torch.Tensor], positions: Optional[torch.Tensor] = None):
    """→ (mixer output [T, width], this layer's values [T, kv_heads, vdim] as they are cached)."""
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T) if positions is None else positions
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(T, H, dk)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(T, G, dk)
    v = unit_rms((h @ w[p + "v"].T).view(T, G, dv), eps)
    if m.get("rot"):
        q, k = rotate_half(q, pos, m["rot"]), rotate_half(k, pos, m["rot"])
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"].reshape(())
        v = (1.0 - lam) * v + lam * v_first
    window = int((m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        lo = max(0, t - window + 1) if window > 0 else 0
        for hd in range(H):
            g = hd // (H // G)
            sc = (k[lo:t + 1, g] @ q[t, hd]) * float(m["scale"])
            out[t, hd] = torch.softmax(sc, 0) @ v[lo:t + 1, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T, v


# -------------------------------------------------------------------------------------------------- generalized delta
def general_delta(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    r, k, v = [(h @ w[p + n].T).view(T, H, d) for n in ("r", "k", "v")]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    a = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=h.dtype)            # [head, key channel, value channel]
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        removed = torch.einsum("hk,hkv->hv", u[t], S)  # uᵀ S of the old state
        S = decay[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * removed[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, r[t])
    o = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# -------------------------------------------------------------------------------------------------------------- mamba2
def mamba2(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dv, N, G, taps = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"])
    parts = int(m.get("norm_groups", 1))
    inner = H * dv
    zz = h @ w[p + "in"].T
    z, xbc, dt = zz[:, :inner], zz[:, inner:2 * inner + 2 * G * N], zz[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc], 0)
    conv = sum(padded[j:j + T] * w[p + "conv"][:, j] for j in range(taps)) + w[p + "conv.b"]
    conv = F.silu(conv)
    x = conv[:, :inner].view(T, H, dv)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w[p + "dt_bias"])             # [T, H]
    rate = torch.exp(w[p + "A_log"])
    S = torch.zeros(H, N, dv, dtype=h.dtype)
    y = torch.zeros(T, H, dv, dtype=h.dtype)
    grp = torch.arange(H) // (H // G)
    for t in range(T):
        Bt, Ct = B[t][grp], C[t][grp]                  # [H, N]
        S = torch.exp(-rate * dt[t])[:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, Ct) + w[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * F.silu(z)
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# -------------------------------------------------------------------------------------------------------- feed-forward
def expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h: torch.Tensor, mlp: dict, router: torch.Tensor):
    """→ (chosen experts [T, top], their weights [T, top])."""
    top = int(mlp["router"]["top"])
    s = torch.softmax(h @ router.T, -1)
    val, idx = torch.sort(s, dim=-1, descending=True, stable=True)
    val, idx = val[:, :top], idx[:, :top]
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * float(mlp["router"]["scale"])


def moe(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    idx, wt = route(h, mlp, w[p + "router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * expert(h[t:t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# --------------------------------------------------------------------------------------------------------- whole model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; `trace` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    v_first = None
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", lc["mixer"]
        if lc["type"] == "attention":
            y, v = attention(x, m, w, p, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif lc["type"] == "general_delta":
            y = general_delta(x, m, w, p, eps)
        elif lc["type"] == "mamba2":
            y = mamba2(x, m, w, p, eps)
        else:
            raise ValueError(lc["type"])
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        if lc.get("mlp") is not None:
            x = x + rms_norm(moe(x, lc["mlp"], w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
