"""A plain, slow statement of the Sefalorn decoder: one function per mechanism, whole sequences at once, on the CPU.

It shares no code with the package: it takes config.json as a dictionary and the tensors by their names, and works in
the dtype it is given (float32, or float64 to bound the float32 one).  A prompt is run whole; there is no cache and
no state that outlives a call, so it cannot have the faults that a cut prompt or a shared batch could bring.

Notation: T tokens, W width, H heads, G key/value heads, D key size, E value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(variance + eps) * w, the variance being the mean of the squared deviations; no bias."""
    c = x - x.mean(dim=-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(dim=-1, keepdim=True) + eps) * w


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def unit_vector(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def residual_gate(h: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """sigmoid(W h + b): what a sub-layer's result is multiplied by before it joins the stream."""
    return torch.sigmoid(h @ w[name].T + w[f"{name}.b"])


# ---- mixers ------------------------------------------------------------------------------------------------------
def fixed_decay_rule(q, k, v, decay, S=None) -> torch.Tensor:
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t for q, k [T, H, D], v [T, H, E], decay [H]; S [H, D, E], if
    given, is where the walk starts and is updated in place."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=q.dtype) if S is None else S
    o = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S.copy_(decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :])
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o


def lightning(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head on silu'd queries, keys and values, walked token by token; the
    heads are normed together."""
    T = h.shape[0]
    H, D, E = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[f"{p}.q"].T).view(T, H, D)
    k = silu(h @ w[f"{p}.k"].T).view(T, H, D)
    v = silu(h @ w[f"{p}.v"].T).view(T, H, E)
    o = fixed_decay_rule(q, k, v, torch.tensor(m["decay"], dtype=torch.float64).to(h.dtype))
    o = rms_unit(o.reshape(T, H * E), eps) * w[f"{p}.norm"]
    return (o * torch.sigmoid(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def mixed_score_attention(q, k, v, positions, scale: float, r1, r2, talk, window: Optional[int]) -> torch.Tensor:
    """Queries q [n, H, D] that stand at ``positions`` over one sequence's keys k [T, G, D] and values v [T, G, E]
    (key j at position j): score = q . k * scale - r1_h ln(1 + r2_h (i - j)); the heads' scores mixed by talk [H, H];
    position i sees 0 <= i - j < window; softmax; values of the head's own group.  [n, H, E]."""
    n, H, _ = q.shape
    G, E = k.shape[1], v.shape[2]
    dist = positions[:, None] - torch.arange(k.shape[0])[None, :]
    see = dist >= 0
    if window is not None:
        see = see & (dist < window)
    far = dist.clamp(min=0).to(q.dtype)
    scores = torch.zeros(H, n, k.shape[0], dtype=q.dtype)
    for head in range(H):
        scores[head] = (q[:, head] @ k[:, head // (H // G)].T) * scale - r1[head] * torch.log(1.0 + r2[head] * far)
    mixed = torch.einsum("hg,gij->hij", talk.to(q.dtype), scores)
    prob = torch.softmax(mixed.masked_fill(~see[None], float("-inf")), dim=-1)
    out = torch.zeros(n, H, E, dtype=q.dtype)
    for head in range(H):
        out[:, head] = prob[head] @ v[:, head // (H // G)]
    return out


def window_attention(h, m: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """Grouped-query attention without rotation: biased projections, a logarithmic penalty on distance, the heads'
    scores mixed by a matrix before the softmax, a sliding window."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[f"{p}.q"].T + w[f"{p}.q.b"]).view(T, H, D)
    k = (h @ w[f"{p}.k"].T + w[f"{p}.k.b"]).view(T, G, D)
    v = (h @ w[f"{p}.v"].T + w[f"{p}.v.b"]).view(T, G, E)
    window = int(m["mask"]["size"]) if m.get("mask") else None      # no mask: every earlier position is seen
    out = mixed_score_attention(q, k, v, torch.arange(T), float(m["scale"]), w[f"{p}.r1"], w[f"{p}.r2"],
                                w[f"{p}.talk"], window)
    return out.reshape(T, H * E) @ w[f"{p}.o"].T + w[f"{p}.o.b"]


def short_conv(x: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """Causal convolution per channel: taps_w [channels, taps], the last column weighs the token itself, zeros stand
    before the start."""
    T, taps = x.shape[0], taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j][None, :]
    return out


def delta_rule(q, k, v, beta, fade, S=None) -> torch.Tensor:
    """Per head: S <- fade_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.  q, k [T, G, D] (head h
    reads group h / (H / G)), v [T, H, E], beta and fade [T, H]; S [H, D, E], if given, is where the walk starts and
    is updated in place."""
    T, G, D = q.shape
    H, E = v.shape[1], v.shape[2]
    group = torch.arange(H) // (H // G)
    S = torch.zeros(H, D, E, dtype=q.dtype) if S is None else S
    o = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        kt, qt = k[t][group], q[t][group]                                            # [H, D]
        S.mul_(fade[t][:, None, None])
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, kt))
        S.add_(kt[:, :, None] * u[:, None, :])
        o[t] = torch.einsum("hde,hd->he", S, qt)
    return o


def gated_delta(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The gated delta rule: a matrix state per head that fades, is corrected towards the value at the key, and is
    read after the write."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_conv(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"])).view(T, H, E)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)                                          # [T, H]
    fade = torch.exp(-torch.exp(w[f"{p}.A_log"]) * softplus(h @ w[f"{p}.a"].T + w[f"{p}.dt_bias"]))
    o = delta_rule(q, k, v, beta, fade)
    o = rms_unit(o, eps) * w[f"{p}.norm"]
    o = o.reshape(T, H * E) * silu(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def parallel(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    return float(m["left_scale"]) * window_attention(h, m["left"], w, f"{p}.left") \
        + float(m["right_scale"]) * gated_delta(h, m["right"], w, f"{p}.right", eps)


# ---- feed-forward ------------------------------------------------------------------------------------------------
def expert(h, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def sigmoid_shares(z: torch.Tensor, top: int, scale: float) -> torch.Tensor:
    """[rows, experts]: for the ``top`` experts with the largest sigmoid(z) their score over the sum of the chosen
    scores (+ 1e-20) times ``scale``, zero for the others."""
    best, chosen = torch.topk(torch.sigmoid(z), top, dim=-1)
    weight = best / (best.sum(dim=-1, keepdim=True) + 1e-20) * scale
    return torch.zeros_like(z).scatter_(1, chosen, weight)


def moe_ff(h, mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """Experts chosen by the largest sigmoid scores, weighed by their scores over the chosen scores' sum, times a
    constant."""
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    share = sigmoid_shares(h @ w[f"{p}.router"].T, top, float(mlp["router"]["scale"]))
    out = torch.zeros_like(h)
    for e in range(n):
        out = out + share[:, e:e + 1] * expert(h, w, f"{p}.e{e}")
    return out


# ---- the model ---------------------------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs``, if a list, receives the residual after each layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        m, kind, p = layer["mixer"], layer["type"], f"l{i}.mix"
        h = layer_norm(x, w[f"l{i}.norm1"], eps)
        if kind == "lightning":
            y = lightning(h, m, w, p, eps)
        elif kind == "parallel":
            y = parallel(h, m, w, p, eps)
        else:
            raise ValueError(f"layer {i}: no mixer '{kind}'")
        x = x + residual_gate(h, w, f"l{i}.rg1") * y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[f"l{i}.norm2"], eps)
            x = x + residual_gate(h, w, f"l{i}.rg2") * moe_ff(h, mlp, w, f"l{i}.mlp")
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T * float(config["logit_scale"])


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=torch.float32) -> List[int]:
    """The tokens that always taking the largest logit gives (the whole sequence is run again for every token)."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, weights, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
