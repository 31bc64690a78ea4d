"""Plain, slow restatement of the Tarudra design in torch on the CPU — one function per mechanism, written from the
design's equations and sharing no code with the package.  It takes the config as the plain dict config.json holds and the
weights under their checkpoint names (as float tensors).

Tarudra: a residual stream x [T, width]; every layer is  x += s1 * LN_b(mixer(LN_a(x)))  then  x += s2 * LN_d(ff(LN_c(x)))
with weight-only layer norms and a per-channel layer scale s.  Mixers: a sliding-window softmax attention with grouped
heads, biases, interleaved rotary pairs under YaRN stretching and a sink in the softmax's denominator, optionally reading
the keys and values an earlier layer cached; a latent attention whose queries and keys / values go through low-rank
latents, with a rotate-half rotary part, a sliding window and a sigmoid output gate; or the gated delta rule behind short
causal convolutions.  The feed-forward is a dense squared-ReLU layer; the logits are capped with a tanh.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------------------- norms
def layer_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    m = v.mean(-1, keepdim=True)
    c = v - m
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w


def rms_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w


# -------------------------------------------------------------------------------------------------------------- rotary
def rotary_frequencies(rot: dict):
    """→ (angular frequency of every pair [dims/2] in float64, the factor cos and sin are multiplied by)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v: torch.Tensor, positions: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
    """v [T, heads, n]: the first rot.dims entries of every head turn with the position; "interleaved" pairs entry 2i with
    2i + 1, "half" pairs entry i with i + dims/2."""
    dims = int(rot["dims"])
    if dims == 0:
        return v
    f, mag = rotary_frequencies(rot)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag).to(v.dtype)[:, None, :], (torch.sin(ang) * mag).to(v.dtype)[:, None, :]
    out = v.clone()
    if layout == "interleaved":
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        h = dims // 2
        a, b = v[..., :h], v[..., h:dims]
        out[..., :h] = a * c - b * s
        out[..., h:dims] = b * c + a * s
    return out


def window_mask(pos_q: torch.Tensor, pos_k: torch.Tensor, size: int) -> torch.Tensor:
    d = pos_q[:, None] - pos_k[None, :]
    return (d >= 0) & ((d < size) if size > 0 else torch.ones_like(d, dtype=torch.bool))


# ----------------------------------------------------------------------------------------------------------- attention
def attention_keys_values(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str):
    """The rotated keys [T, kv_heads, dim] and the values [T, kv_heads, vdim] a layer with projections of its own caches."""
    T, G, dk, dv = h.shape[0], int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = (h @ w[p + "mix.k"].T + w[p + "mix.k.b"]).view(T, G, dk)
    v = (h @ w[p + "mix.v"].T + w[p + "mix.v.b"]).view(T, G, dv)
    if m.get("rot"):
        k = rotate(k, positions, m["rot"], "interleaved")
    return k, v


def attention(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, keys: torch.Tensor,
              values: torch.Tensor, key_positions: torch.Tensor, sink: bool = True) -> torch.Tensor:
    """Windowed attention of the rows h over (keys, values) at key_positions; the softmax has a sink: 1 is added to its
    denominator (sink=False: an ordinary softmax, for tests that show the sink matters)."""
    T, H, G, dk, dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "mix.q"].T + w[p + "mix.q.b"]).view(T, H, dk)
    if m.get("rot"):
        q = rotate(q, positions, m["rot"], "interleaved")
    vis = window_mask(positions, key_positions, int((m.get("mask") or {}).get("size", 0)))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ keys[:, g].T) * float(m["scale"])
        s = s.masked_fill(~vis, float("-inf"))
        mx = s.max(-1, keepdim=True).values.clamp_min(0.0)
        e = torch.exp(s - mx)
        out[:, hd] = (e / ((torch.exp(-mx) if sink else 0.0) + e.sum(-1, keepdim=True))) @ values[:, g]
    return out.reshape(T, H * dv) @ w[p + "mix.o"].T + w[p + "mix.o.b"]


# ---------------------------------------------------------------------------------------------------- latent attention
def latent_cache_rows(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """What a latent-attention layer caches per token: the normed latent [T, kv_rank] and the rotated shared key part."""
    r = int(m["kv_rank"])
    down = h @ w[p + "mix.dkv"].T
    c = rms_norm(down[:, :r], w[p + "mix.dkv.norm"], eps)
    kr = down[:, r:]
    if m.get("rot") and int(m["rot_dim"]) > 0:
        kr = rotate(kr[:, None, :], positions, m["rot"], "half")[:, 0]
    return c, kr


def latent_attention(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float,
                     c: torch.Tensor, kr: torch.Tensor, key_positions: torch.Tensor) -> torch.Tensor:
    T, H, dn, dr, dv = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    cq = rms_norm(h @ w[p + "mix.dq"].T, w[p + "mix.dq.norm"], eps)
    q = (cq @ w[p + "mix.uq"].T).view(T, H, dn + dr)
    qn, qr = q[..., :dn], q[..., dn:]
    if m.get("rot") and dr > 0:
        qr = rotate(qr, positions, m["rot"], "half")
    kn = (c @ w[p + "mix.uk"].T).view(-1, H, dn)
    vv = (c @ w[p + "mix.uv"].T).view(-1, H, dv)
    vis = window_mask(positions, key_positions, int((m.get("mask") or {}).get("size", 0)))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * float(m["scale"])
        s = s.masked_fill(~vis, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ vv[:, hd]
    gate = torch.sigmoid(h @ w[p + "mix.g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "mix.o"].T


# ---------------------------------------------------------------------------------------------------- gated delta rule
def short_conv(x: torch.Tensor, taps: torch.Tensor, before: Optional[torch.Tensor]):
    """x [T, C], taps [C, n] (last column meets the current token), before [n − 1, C] or None (zeros) → (y [T, C], the last
    n − 1 inputs)."""
    n = taps.shape[1]
    if before is None:
        before = torch.zeros(n - 1, x.shape[1], dtype=x.dtype)
    full = torch.cat([before, x], 0)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        y[t] = (full[t:t + n] * taps.T).sum(0)
    return y, full[full.shape[0] - (n - 1):]


def delta_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float, state: Optional[dict]):
    """The gated delta rule over the rows h, token by token.  state: {"S": [heads, dim, vdim], "q", "k", "v": the
    convolutions' last inputs} or None (a fresh sequence) → (output [T, width], new state)."""
    T, H, G, dk, dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    st = state or {}
    q, cq = short_conv(h @ w[p + "mix.q"].T, w[p + "mix.q.conv"], st.get("q"))
    k, ck = short_conv(h @ w[p + "mix.k"].T, w[p + "mix.k.conv"], st.get("k"))
    v, cv = short_conv(h @ w[p + "mix.v"].T, w[p + "mix.v.conv"], st.get("v"))
    q, k, v = F.silu(q).view(T, G, dk), F.silu(k).view(T, G, dk), F.silu(v).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "mix.b"].T)
    decay = torch.exp(-torch.exp(w[p + "mix.A_log"]) * F.softplus(h @ w[p + "mix.a"].T + w[p + "mix.dt_bias"]))
    S = st["S"].clone() if "S" in st else torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            o[t, hd] = S[hd].T @ q[t, g]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w[p + "mix.norm"]
    o = o.reshape(T, H * dv) * F.silu(h @ w[p + "mix.g"].T)
    return o @ w[p + "mix.o"].T, {"S": S, "q": cq, "k": ck, "v": cv}


# -------------------------------------------------------------------------------------------------------- feed-forward
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return torch.relu(h @ w[p + "mlp.up"].T) ** 2 @ w[p + "mlp.down"].T


# --------------------------------------------------------------------------------------------------------- whole model
class Sequence:
    """One sequence's memory: what every layer keeps between calls (rows of keys / values or latents, or a state)."""

    def __init__(self, cfg: dict):
        self.n = 0
        self.mem: List[dict] = [{} for _ in cfg["layers"]]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, seq: Optional[Sequence] = None, layer_outputs: Optional[list] = None,
            sink: bool = True):
    """Logits [T, vocab] of the new tokens of one sequence; `seq` carries the memory of the earlier ones."""
    seq = seq if seq is not None else Sequence(cfg)
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    positions = torch.arange(seq.n, seq.n + T)
    x = w["embed"][ids]
    for i, lc in enumerate(cfg["layers"]):
        p, m, mem = f"l{i}.", lc["mixer"], seq.mem[i]
        h = layer_norm(x, w[p + "norm1"], eps)
        if lc["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                k, v = attention_keys_values(h, positions, m, w, p)
                mem["k"] = torch.cat([mem["k"], k], 0) if "k" in mem else k
                mem["v"] = torch.cat([mem["v"], v], 0) if "v" in mem else v
                src = i
            keys, values = seq.mem[int(src)]["k"], seq.mem[int(src)]["v"]
            y = attention(h, positions, m, w, p, keys, values, torch.arange(keys.shape[0]), sink=sink)
        elif lc["type"] == "latent_attention":
            c, kr = latent_cache_rows(h, positions, m, w, p, eps)
            mem["c"] = torch.cat([mem["c"], c], 0) if "c" in mem else c
            mem["kr"] = torch.cat([mem["kr"], kr], 0) if "kr" in mem else kr
            y = latent_attention(h, positions, m, w, p, eps, mem["c"], mem["kr"], torch.arange(mem["c"].shape[0]))
        elif lc["type"] == "delta":
            y, new = delta_mixer(h, m, w, p, eps, mem.get("state"))
            mem["state"] = new
        else:
            raise ValueError(lc["type"])
        x = x + layer_norm(y, w[p + "norm1b"], eps) * w[p + "ls1"]
        if lc.get("mlp") is not None:
            y = dense_ff(layer_norm(x, w[p + "norm2"], eps), w, p)
            x = x + layer_norm(y, w[p + "norm2b"], eps) * w[p + "ls2"]
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    seq.n += T
    z = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap > 0 else z


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt, steps: int) -> List[int]:
    seq = Sequence(cfg)
    out, z = [], forward(cfg, w, prompt, seq)
    for _ in range(steps):
        out.append(int(z[-1].argmax()))
        z = forward(cfg, w, [out[-1]], seq)
    return out
