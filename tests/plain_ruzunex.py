"""A plain, slow statement of the Ruzunex decoder: one function per mechanism, whole sequences at once, on the CPU.

It shares no code with the package: it takes config.json as a dictionary and the tensors by their names, and works in
the dtype it is given (float32, or float64 to bound the float32 one).  A prompt is run whole; there is no cache and
no state that outlives a call, so it cannot have the faults that a cut prompt or a shared batch could bring.

Notation: T tokens, W width, S streams, H heads, G key/value heads, D key size, E value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last dimension (w None: the division alone)."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """y_t = sum_j w[:, j] x_(t - taps + 1 + j) per channel: x [T, C], taps_w [C, taps]; the last column weighs the
    token itself, zeros stand before the start."""
    T, taps = x.shape[0], taps_w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += taps_w[:, j] * x[s]
    return out


# ---- the residual of several streams ---------------------------------------------------------------------------
def streams_read(x: torch.Tensor, read: torch.Tensor) -> torch.Tensor:
    """u = sum_s read[s] x_s for x [T, S, W]."""
    return torch.einsum("s,tsw->tw", read, x)


def streams_update(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, gain: torch.Tensor) -> torch.Tensor:
    """x_t <- sum_s mix[s, t] x_s + gain[t] y, all streams at once from the old ones."""
    return torch.einsum("sr,tsw->trw", mix, x) + gain[None, :, None] * y[:, None, :]


# ---- attention ---------------------------------------------------------------------------------------------------
def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: the first ``dims`` numbers of every head turn by position, number i with number i + dims/2;
    pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).to(torch.float32 if x.dtype != torch.float64 else torch.float64)
    ang = positions.to(freq.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def attention_scores(q: torch.Tensor, k: torch.Tensor, scale: float) -> torch.Tensor:
    """[H, T, T] scaled products of queries q [T, H, D] with the keys k [T, G, D] of each head's group."""
    H, G = q.shape[1], k.shape[1]
    return torch.stack([(q[:, h] @ k[:, h // (H // G)].T) * scale for h in range(H)])


def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """[T, T]: position i sees j with 0 <= i - j (< window, if there is one)."""
    dist = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    see = dist >= 0
    return see & (dist < window) if window is not None else see


def weighted_values(prob: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """prob [H, T, T], v [T, G, E] -> [T, H * E]."""
    H, G = prob.shape[0], v.shape[1]
    return torch.cat([prob[h] @ v[:, h // (H // G)] for h in range(H)], dim=-1)


def sliding_attention(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float,
                      v_first: Optional[torch.Tensor]):
    """The mixer "attention": norms per head on queries and keys, no rotation, a bias slope_h (i - j) taken off the
    scores, a sliding window, values blended with the first such layer's, a sigmoid gate on the heads.  Returns the
    output and the values as they are cached."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_norm((h @ w[f"{p}.q"].T).view(T, H, D), w[f"{p}.q.norm"], eps)
    k = rms_norm((h @ w[f"{p}.k"].T).view(T, G, D), w[f"{p}.k.norm"], eps)
    v = (h @ w[f"{p}.v"].T).view(T, G, E)
    if v_first is not None:
        lam = w[f"{p}.vmix"]
        v = (1.0 - lam) * v + lam * v_first
    s = attention_scores(q, k, float(m["scale"]))
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).to(h.dtype)
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=torch.float64).to(h.dtype)
    s = s - slopes[:, None, None] * dist[None]
    window = int(m["mask"]["size"]) if m.get("mask") else None
    prob = torch.softmax(s.masked_fill(~visible(T, window)[None], float("-inf")), dim=-1)
    o = weighted_values(prob, v) * torch.sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T, v


def sink_softmax(s: torch.Tensor, see: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Softmax over the visible keys whose denominator also holds exp(sink_h): s [H, T, T], sink [H]."""
    s = s.masked_fill(~see[None], float("-inf"))
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def sink_attention(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The left half of the mixer "parallel": short convolutions behind the projections, norms over the whole
    projection, partial rotation, a factor per head on the scores, every earlier key visible, a sink in the
    softmax."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = causal_conv(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"])
    k = causal_conv(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"])
    v = causal_conv(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"])
    q = rms_norm(q, w[f"{p}.q.norm"], eps).view(T, H, D)
    k = rms_norm(k, w[f"{p}.k.norm"], eps).view(T, G, D)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, int(rot["dims"]), float(rot["base"]))
        k = rotate_half(k, pos, int(rot["dims"]), float(rot["base"]))
    s = attention_scores(q, k, float(m["scale"])) * w[f"{p}.temp"][:, None, None]
    window = int(m["mask"]["size"]) if m.get("mask") else None      # no mask: every earlier position is seen
    prob = sink_softmax(s, visible(T, window), w[f"{p}.sink"])
    return weighted_values(prob, v.view(T, G, E)) @ w[f"{p}.o"].T


# ---- the recurrent half ------------------------------------------------------------------------------------------
def forget_write_rule(q, f, v, S=None) -> torch.Tensor:
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t for q, f [T, H, D], v [T, H, E]; S [H, D, E], if
    given, is where the walk starts and is updated in place."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=q.dtype) if S is None else S
    o = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S.copy_(f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :])
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o


def forget_write_mixer(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The right half of the mixer "parallel": a forget gate with a learned lower bound whose complement says what is
    written; every head's result normed over its value size with one shared weight."""
    T = h.shape[0]
    H, D, E = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[f"{p}.q"].T).view(T, H, D)
    v = (h @ w[f"{p}.v"].T).view(T, H, E)
    low = w[f"{p}.lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[f"{p}.f"].T + w[f"{p}.f.b"])).view(T, H, D)
    o = rms_norm(forget_write_rule(q, f, v), w[f"{p}.norm"], eps)
    return o.reshape(T, H * E) @ w[f"{p}.o"].T


# ---- feed-forward ------------------------------------------------------------------------------------------------
def dense_ff(h, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def expert_ff(h, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[f"{p}.gate"].T, max=limit)
    u = torch.clamp(h @ w[f"{p}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{p}.down"].T


def route(z: torch.Tensor, top: int):
    """Scores by softmax over all experts; the ``top`` largest are chosen (equal scores: the lower index) and weighed
    by their share of the chosen scores.  Returns (indices [T, top], weights [T, top])."""
    s = torch.softmax(z, dim=-1)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    chosen = torch.gather(s, 1, order)
    return order, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def routed_ff(h, mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    idx, wt = route((h @ w[f"{p}.router"].T).to(h.dtype), int(mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            out[t] += a * expert_ff(h[t:t + 1], w, f"{p}.e{e}", float(mlp["expert"]["limit"]))[0]
    return out


# ---- the model ---------------------------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32,
            layer_sums: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``layer_sums``: a list that receives the sum of the streams after every
    layer."""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    S = int(config["streams"])
    e = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = e[:, None, :].repeat(1, S, 1)
    v_first = None
    seen_v_mix = False
    for i, layer in enumerate(config["layers"]):
        m, L = layer["mixer"], f"l{i}"
        u = rms_norm(streams_read(x, w[f"{L}.hc1.in"]), w[f"{L}.norm1"], eps)
        u = u + causal_conv(u, w[f"{L}.canon1"])
        if layer["type"] == "attention":
            blend = bool(m.get("v_mix")) and seen_v_mix
            y, v = sliding_attention(u, m, w, f"{L}.mix", eps, v_first if blend else None)
            if m.get("v_mix") and not seen_v_mix:
                v_first, seen_v_mix = v, True
        elif layer["type"] == "parallel":
            y = float(m["left_scale"]) * sink_attention(u, m["left"], w, f"{L}.mix.left", eps) \
                + float(m["right_scale"]) * forget_write_mixer(u, m["right"], w, f"{L}.mix.right", eps)
        else:
            raise ValueError(layer["type"])
        x = streams_update(x, y, w[f"{L}.hc1.mix"], w[f"{L}.hc1.out"])
        mlp = layer.get("mlp")
        if mlp is not None:
            u = rms_norm(streams_read(x, w[f"{L}.hc2.in"]), w[f"{L}.norm2"], eps)
            u = u + causal_conv(u, w[f"{L}.canon2"])
            y = dense_ff(u, w, f"{L}.mlp") if mlp["kind"] == "dense" else routed_ff(u, mlp, w, f"{L}.mlp")
            x = streams_update(x, y, w[f"{L}.hc2.mix"], w[f"{L}.hc2.out"])
        if layer_sums is not None:
            layer_sums.append(x.sum(dim=1))
    return rms_norm(x.sum(dim=1), w["final.norm"], eps) @ w["head"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=torch.float32) -> List[int]:
    """The tokens that the largest logit picks, one after the other, the whole sequence run again for each."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, weights, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
