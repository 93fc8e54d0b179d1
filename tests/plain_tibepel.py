"""Plain, slow implementation of the Tibepel decoder, used as the oracle of its tests.

Whole sequences only: no cache, no state carried between calls, no batching; one function per
mechanism, torch used purely as an array library (float64 on the CPU).  It shares no code with the
engine under ``rvllm_b200``: the configuration is a plain dictionary and the weights a plain dictionary
name -> tensor.  `store`, where a function has it, is applied to what an engine keeps between two kernels
in the activations' type (the identity, or a rounding to bfloat16 that measures what that storage costs).

The design in this file's notation (h: a sublayer's input; W x: a matrix stored [out, in] applied to a
column; n(v) = v / sqrt(mean(v^2) + eps)):

* input:     x = embed[token] * s_e + pe(p);  pe(p)[2i] = sin(p w_i), pe(p)[2i+1] = cos(p w_i), w_i = 10000^(-2i/width);
* a layer:   x <- x + mixer(n(x) (1 + w1));  x <- x + ff(n(x) (1 + w2));  then the token's own side input:
             e = the layer's slice of side_embed[token];  y = P (gelu_tanh(G x) * e);  x <- x + n(y) w_s;
* mamba1:    [u | z] = W_in h;  u <- silu(conv(u) + b);  [d | B | C] = W_x u;  dt = softplus(W_dt d + b_dt);
             S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n  with A = -exp(A_log);  y_c = sum_n S[c, n] C_n + D_c u_c;
             out = W_o (y * silu(z));
* parallel:  a_l * left(h) + a_r * right(h);
  left:      q, k, v with biases; v <- n(v) per head (no weight); s_h(i, j) = c (q_h(i) . k(j)) - r1_h ln(1 + r2_h (i - j)),
             j <= i and floor(i / m) = floor(j / m); p = softmax(s); p'_h = sum_g T[h, g] p_g; o_h = sum_j p'_h(i, j) v(j);
             out = W_o o + b_o;
  right:     q, k, v <- silu(conv(W h)) (no bias); q, k <- unit vectors per head (q also times dim^-1/2);
             beta = sigmoid(W_b h); g = exp(-exp(A_log) softplus(W_a h + dt_bias));
             S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;  out = W_o (n(o) w * silu(W_g h));
* ff:        g = min(W_g h + b, L);  u = clamp(W_u h + b, -L, L);  out = W_d (g sigmoid(1.702 g) (u + 1)) + b;
* output:    logits = c tanh(head (n(x) (1 + w_f)) / c).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


def _keep(t: torch.Tensor) -> torch.Tensor:
    return t


def round_to_bfloat16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def sinusoid(positions: Sequence[int], width: int) -> torch.Tensor:
    """[T, width]: entry 2i is the sine, entry 2i + 1 the cosine of p * 10000^(-2i / width)."""
    out = torch.zeros((len(positions), width), dtype=F64)
    for row, p in enumerate(positions):
        for i in range((width + 1) // 2):
            a = p * 10000.0 ** (-2.0 * i / width)
            out[row, 2 * i] = math.sin(a)
            if 2 * i + 1 < width:
                out[row, 2 * i + 1] = math.cos(a)
    return out


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """u [T, C], taps [C, K] (column K - 1 multiplies the current token), zeros before the sequence."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros((K - 1, C), dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j][None, :]
    return out if bias is None else out + bias[None, :]


# ---------------------------------------------------------------------------------------------- mamba1
def channel_scan(u, dt, A, B, C, D) -> torch.Tensor:
    """u, dt [T, inner]; A [inner, N]; B, C [T, N]; D [inner] -> y [T, inner].  One state row per channel."""
    T, inner = u.shape
    S = torch.zeros((inner, A.shape[1]), dtype=u.dtype)
    y = torch.zeros_like(u)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y


def mamba1_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, store=_keep) -> torch.Tensor:
    inner, N, r = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].t()
    u, z = xz[:, :inner], xz[:, inner:]
    u = store(silu(causal_conv(u, w[p + "conv"], w[p + "conv.b"])))
    dbc = u @ w[p + "x"].t()
    d, B, C = dbc[:, :r], dbc[:, r:r + N], dbc[:, r + N:]
    dt = softplus(store(d) @ w[p + "dt"].t() + w[p + "dt.b"])
    y = channel_scan(u, dt, -torch.exp(w[p + "A_log"]), B, C, w[p + "D"])
    return store(y * silu(z)) @ w[p + "o"].t()


# ---------------------------------------------------------------------------------------------- left: attention
def mixed_head_attention(q, k, v, scale: float, r1, r2, talk, chunk: int, start: int = 0) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv], r1, r2 [H], talk [H, H] -> [T, H, dv].

    Every head's softmax weights over the keys of its chunk are formed first, with the logarithmic
    penalty of the distance; then head h's weights become a combination of all heads' weights (row h of
    `talk`), and those act on the values of h's own key/value head."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for t in range(T):
        i = start + t
        lo = (i // chunk) * chunk - start          # first visible key of the chunk, as an index into k
        lo = max(lo, 0)
        dist = torch.arange(t - lo, -1, -1, dtype=q.dtype)       # i - j for j = lo .. t
        P = torch.zeros((H, t + 1 - lo), dtype=q.dtype)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:t + 1, g] @ q[t, h]) * scale - r1[h] * torch.log1p(r2[h] * dist)
            P[h] = torch.softmax(s, dim=0)
        Pm = talk @ P
        for h in range(H):
            g = h // (H // G)
            out[t, h] = Pm[h] @ v[lo:t + 1, g]
    return out


def left_mixer(h, w, p: str, m: dict, eps: float, start: int = 0, store=_keep) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ w[p + "q"].t() + w[p + "q.b"]).view(T, H, d)
    k = store(h @ w[p + "k"].t() + w[p + "k.b"]).view(T, G, d)
    v = store(rms((h @ w[p + "v"].t() + w[p + "v.b"]).view(T, G, dv), eps))
    o = mixed_head_attention(q, k, v, m["scale"], w[p + "r1"], w[p + "r2"], w[p + "talk"], m["mask"]["size"], start)
    return store(o).reshape(T, -1) @ w[p + "o"].t() + w[p + "o.b"]


# ---------------------------------------------------------------------------------------------- right: gated delta rule
def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """q, k [T, H, d] (already per value head), v [T, H, dv], beta, g [T, H] -> o [T, H, dv]."""
    T, H, d = q.shape
    S = torch.zeros((H, d, v.shape[2]), dtype=q.dtype)
    o = torch.zeros_like(v)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def right_mixer(h, w, p: str, m: dict, eps: float, store=_keep) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(silu(causal_conv(h @ w[p + "q"].t(), w[p + "q.conv"], None))).view(T, G, d)
    k = store(silu(causal_conv(h @ w[p + "k"].t(), w[p + "k.conv"], None))).view(T, G, d)
    v = store(silu(causal_conv(h @ w[p + "v"].t(), w[p + "v.conv"], None))).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].t())
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].t() + w[p + "dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    gate = silu(h @ w[p + "g"].t()).view(T, H, dv)
    o = rms(o, eps) * w[p + "norm"][None, None, :] * gate
    return store(o).reshape(T, -1) @ w[p + "o"].t()


def parallel_mixer(h, w, p: str, m: dict, eps: float, start: int = 0, store=_keep) -> torch.Tensor:
    return m["left_scale"] * left_mixer(h, w, p + "left.", m["left"], eps, start, store) + \
        m["right_scale"] * right_mixer(h, w, p + "right.", m["right"], eps, store)


# ---------------------------------------------------------------------------------------------- feed-forward, side input
def clamped_glu(h, w, p: str, limit: float, store=_keep) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].t() + w[p + "gate.b"], max=limit)
    u = torch.clamp(h @ w[p + "up"].t() + w[p + "up.b"], min=-limit, max=limit)
    return store(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].t() + w[p + "down.b"]


def side_input(x, tokens: Sequence[int], w, p: str, layer: int, dim: int, eps: float, store=_keep) -> torch.Tensor:
    e = w["side.embed"][list(tokens)][:, layer * dim:(layer + 1) * dim]
    g = store(gelu_tanh(store(x) @ w[p + "gate"].t()) * e)
    y = g @ w[p + "proj"].t()
    return rms(y, eps) * w[p + "norm"]


# ---------------------------------------------------------------------------------------------- the model
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], store=_keep, layers_out: Optional[List] = None,
            start: int = 0) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence.  `layers_out`, a list, receives the stream after every layer."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = w["embed"][list(tokens)] * cfg["embedding"]["scale"] + sinusoid(range(start, start + T), cfg["width"])
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = store(offset_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "mamba1":
            x = x + mamba1_mixer(h, w, p + "mix.", layer["mixer"], store)
        else:
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, start, store)
        if layer.get("mlp") is not None:
            h = store(offset_norm(x, w[p + "norm2"], eps))
            x = x + clamped_glu(h, w, p + "mlp.", layer["mlp"]["limit"], store)
        if side is not None:
            x = x + side_input(x, tokens, w, p + "side.", i, side["dim"], eps, store)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = store(offset_norm(x, w["final.norm"], eps))
    logits = h @ w["head"].t()
    cap = cfg.get("logit_softcap")
    return logits if cap is None else cap * torch.tanh(logits / cap)
