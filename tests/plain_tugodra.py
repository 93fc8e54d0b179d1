"""The Tugodra design written out plainly: float64, whole sequences, no cache and no carried state, one function per
mechanism.

It shares nothing with the package: the tests compare the engine (its step function, cache, state rows, kernels) with
this.  Notation: h a sublayer's input [T, width]; u(v) = v / sqrt(mean(v^2) + eps) over the last dimension.

`store` is applied to every tensor that an engine keeps between two kernels (identity by default; `round_to_bfloat16`
measures what bfloat16 storage costs by itself, all arithmetic staying float64).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def _keep(t):
    return t


def round_to_bfloat16(t):
    return t.to(torch.bfloat16).to(torch.float64)


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def dynamic_tanh(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """tanh(alpha x) * weight + bias, element by element: no statistic of the row is formed."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def _angles(positions: torch.Tensor, i: int, dims: int, base: float):
    ang = positions.to(torch.float64) * (float(base) ** (-2.0 * i / dims))
    return torch.cos(ang), torch.sin(ang)


def turn_neighbours(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, ..., D]: the pairs (2i, 2i + 1), i < dims / 2, turn by position * base^(-2i / dims); the rest stays."""
    out = v.clone()
    shape = [v.shape[0]] + [1] * (v.dim() - 2)
    for i in range(dims // 2):
        c, s = (t.reshape(shape) for t in _angles(positions, i, dims, base))
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def turn_halves(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, ..., D]: the pairs (i, i + dims / 2), i < dims / 2, turn by position * base^(-2i / dims); the rest stays."""
    out = v.clone()
    shape = [v.shape[0]] + [1] * (v.dim() - 2)
    half = dims // 2
    for i in range(half):
        c, s = (t.reshape(shape) for t in _angles(positions, i, dims, base))
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * c - b * s
        out[..., i + half] = b * c + a * s
    return out


def window_keys(h, w, p: str, m: dict, eps: float, positions, store=_keep):
    """What an attention layer leaves for itself and for the layers that borrow from it: keys after the rotation and the
    unit norm, and values."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = turn_neighbours((h @ w[p + "k"].T).reshape(T, G, D), positions, m["rot"]["dims"], m["rot"]["base"])
    return store(unit_rms(k, eps)), store((h @ w[p + "v"].T).reshape(T, G, V))


def window_attention(h, w, p: str, m: dict, eps: float, positions, keys, values, store=_keep) -> torch.Tensor:
    """Grouped heads over `keys` [T, G, D] and `values` [T, G, V] (the layer's own or another layer's); a query sees itself
    and the `mask.size - 1` positions before it; one sigmoid gate per head on the result."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = turn_neighbours((h @ w[p + "q"].T).reshape(T, H, D), positions, m["rot"]["dims"], m["rot"]["base"])
    q = store(unit_rms(q, eps))
    gate = torch.sigmoid(h @ w[p + "g"].T)
    dist = positions[:, None] - positions[None, :]
    hidden = dist < 0
    if m.get("mask") and m["mask"].get("size") is not None:
        hidden = hidden | (dist >= m["mask"]["size"])
    heads = []
    for i in range(H):
        g = i // (H // G)
        score = (q[:, i] @ keys[:, g].T) * m["scale"]
        score = score.masked_fill(hidden, float("-inf"))
        heads.append(store(torch.softmax(score, -1) @ values[:, g] * gate[:, i:i + 1]))
    return torch.cat(heads, dim=1) @ w[p + "o"].T


def latent_attention(h, w, p: str, m: dict, eps: float, positions, store=_keep) -> torch.Tensor:
    """Keys and values of every head from one latent per token, written head by head (nothing absorbed); causal; the
    softmax's denominator also holds exp(sink) of the head."""
    T = h.shape[0]
    H, D, Rd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    q = (h @ w[p + "q"].T).reshape(T, H, D + Rd)
    down = h @ w[p + "dkv"].T
    c = store(unit_rms(down[:, :R], eps) * w[p + "dkv.norm"])
    shared_key = store(turn_halves(down[:, R:], positions, dims, base))
    hidden = positions[None, :] > positions[:, None]
    heads = []
    for i in range(H):
        k_plain = c @ w[p + "uk"][i * D:(i + 1) * D].T
        value = c @ w[p + "uv"][i * V:(i + 1) * V].T
        q_plain = store(q[:, i, :D])
        q_turned = store(turn_halves(q[:, i, D:], positions, dims, base))
        score = (q_plain @ k_plain.T + q_turned @ shared_key.T) * m["scale"]
        score = score.masked_fill(hidden, float("-inf"))
        top = torch.maximum(score.max(-1, keepdim=True).values, w[p + "sink"][i])
        e = torch.exp(score - top)
        weight = e / (e.sum(-1, keepdim=True) + torch.exp(w[p + "sink"][i] - top))
        heads.append(store(weight @ value))
    return torch.cat(heads, dim=1) @ w[p + "o"].T


def mlstm(h, w, p: str, m: dict, eps: float, store=_keep) -> torch.Tensor:
    """A matrix memory per head, walked token by token from an empty state; the running maximum starts at 0."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = store((h @ w[p + "q"].T).reshape(T, H, D)) * D ** -0.5
    k = store((h @ w[p + "k"].T).reshape(T, H, D))
    v = store((h @ w[p + "v"].T).reshape(T, H, V))
    log_in = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    log_keep = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros((T, H, V), dtype=h.dtype)
    for i in range(H):
        S = torch.zeros((D, V), dtype=h.dtype)
        n = torch.zeros((D,), dtype=h.dtype)
        top = 0.0
        for t in range(T):
            new_top = max(float(log_keep[t, i]) + top, float(log_in[t, i]))
            keep, take = math.exp(float(log_keep[t, i]) + top - new_top), math.exp(float(log_in[t, i]) - new_top)
            S = keep * S + take * torch.outer(k[t, i], v[t, i])
            n = keep * n + take * k[t, i]
            top = new_top
            out[t, i] = (S.T @ q[t, i]) / (max(abs(float(n @ q[t, i])), math.exp(-top)) + 1e-6)
    y = (unit_rms(out, eps).reshape(T, H * V) * w[p + "norm"]) * torch.sigmoid(h @ w[p + "g"].T)
    return store(y) @ w[p + "o"].T


def expert(h, w, p: str, store=_keep) -> torch.Tensor:
    return store(torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def route(h, w, p: str, router: dict):
    """Per token the chosen experts and their weights: sigmoid scores; the choice adds a correction per expert and is
    limited to the best groups of neighbouring experts (a group counts by its two largest corrected scores); the
    weights are the uncorrected scores of the chosen, made to sum to one."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ w[p + "router"].T)
    c = s + w[p + "correction"]
    per = E // groups["count"]
    by_group = c.reshape(-1, groups["count"], per)
    group_score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(groups["keep"], dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
    c = c.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    chosen = c.topk(top, dim=-1).indices
    weights = s.gather(1, chosen)
    return chosen, weights / (weights.sum(-1, keepdim=True) + 1e-20)


def moe(h, w, p: str, mlp: dict, store=_keep) -> torch.Tensor:
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", store)[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.", store)
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], store=_keep, streams: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab]; `streams` collects the residual stream after every layer."""
    w = {k: (v.to(torch.float64) if v.is_floating_point() else v.long()) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    pos = torch.arange(len(tok))
    x = w["embed"][tok] * float(cfg["embedding"]["scale"])
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = store(dynamic_tanh(x, w, p + "norm1"))
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = window_keys(h, w, p + "mix.", m, eps, pos, store)
            keys, values = kept[i if m.get("kv_from") is None else m["kv_from"]]
            y = window_attention(h, w, p + "mix.", m, eps, pos, keys, values, store)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", m, eps, pos, store)
        elif layer["type"] == "mlstm":
            y = mlstm(h, w, p + "mix.", m, eps, store)
        else:
            raise ValueError(layer["type"])
        x = x + dynamic_tanh(y, w, p + "norm1b")
        if layer.get("mlp"):
            y = moe(store(dynamic_tanh(x, w, p + "norm2")), w, p + "mlp.", layer["mlp"], store)
            x = x + dynamic_tanh(y, w, p + "norm2b")
        if streams is not None:
            streams.append(x.clone())
    return store(dynamic_tanh(x, w, "final.norm")) @ w["head"].T


def greedy(cfg: dict, weights, prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(torch.argmax(forward(cfg, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
