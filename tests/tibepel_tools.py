"""Small Tibepel configurations, model folders for them and plain logits, for the tests of that design.

The sizes differ from layer to layer and between the configurations and avoid values that hide a fault: value sizes
unlike the key sizes, groups of query heads larger than one on both sides, chunk sizes that are no multiples of a page,
three and five taps, a state size that is no multiple of a warp, a layer without a feed-forward, both orders of the two
kinds of layer, scales of the two sides that differ."""
from __future__ import annotations

import copy
from typing import Dict, List

import torch

import plain_tibepel as P
from tufirax_tools import read_folder, write_folder      # (folders are written by the framework's random-weights mode)


def ff(width=56, limit=1.5):
    return {"kind": "dense", "ff": width, "limit": limit}


def mamba1(inner=40, state=12, dt_rank=5, conv=3, mlp=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": copy.deepcopy(mlp)}


def parallel(heads=6, kv_heads=3, dim=16, vdim=24, scale=0.3, chunk=21, r_heads=4, r_kv=2, r_dim=12, r_vdim=20, r_conv=3,
             left_scale=0.7, right_scale=1.2, mlp=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}},
                      "left_scale": left_scale,
                      "right": {"heads": r_heads, "kv_heads": r_kv, "dim": r_dim, "vdim": r_vdim, "conv": r_conv},
                      "right_scale": right_scale},
            "mlp": copy.deepcopy(mlp)}


def config(layers: List[dict], width=48, vocab=131, eps=1e-5, emb_scale=3.0, cap=20.0, side=6) -> dict:
    c = {"architecture": "Tibepel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
         "layers": copy.deepcopy(layers)}
    if cap is not None:
        c["logit_softcap"] = cap
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


def small_a() -> dict:
    """The scan first, then two side-by-side layers with different sizes (chunks of 21 and of 50 positions: neither a
    multiple of a page), the second without a feed-forward, then another scan with five taps."""
    return config([mamba1(mlp=ff()),
                   parallel(mlp=ff(40, 0.8)),
                   parallel(heads=4, kv_heads=1, dim=24, vdim=8, scale=0.2, chunk=50, r_heads=3, r_kv=3, r_dim=20, r_vdim=12, r_conv=5,
                            left_scale=1.1, right_scale=0.4, mlp=None),
                   mamba1(inner=72, state=33, dt_rank=7, conv=5, mlp=ff(64, 2.5))])


def small_b() -> dict:
    """Side-by-side layers first; sizes of 16-byte rows (keys of 64 and values of 32, a delta rule of 64 x 48 and one of
    128 x 32), a chunk that is a multiple of the page, no cap on the logits, no token side input."""
    return config([parallel(heads=8, kv_heads=2, dim=64, vdim=32, scale=0.11, chunk=32, r_heads=4, r_kv=2, r_dim=64, r_vdim=48, r_conv=4,
                            mlp=ff(96, 1.0)),
                   mamba1(inner=128, state=16, dt_rank=8, conv=4, mlp=None),
                   parallel(heads=2, kv_heads=2, dim=32, vdim=64, scale=0.2, chunk=64, r_heads=2, r_kv=1, r_dim=128, r_vdim=32, r_conv=2,
                            left_scale=0.5, right_scale=0.5, mlp=ff(80, 3.0))],
                  width=64, vocab=203, eps=1e-6, emb_scale=1.0, cap=None, side=None)


def odd_shapes() -> dict:
    """Sizes that no fast path is made for: a width and a vocabulary that are no multiples of 8 (an odd width: the last
    sine has no cosine), one head, odd head and value sizes, a chunk of one position and one far longer than any prompt,
    one tap, a state of one."""
    return config([parallel(heads=1, kv_heads=1, dim=9, vdim=7, scale=0.4, chunk=1, r_heads=1, r_kv=1, r_dim=5, r_vdim=3, r_conv=1,
                            mlp=ff(30, 0.5)),
                   mamba1(inner=11, state=1, dt_rank=1, conv=1, mlp=None),
                   parallel(heads=5, kv_heads=5, dim=10, vdim=11, scale=0.25, chunk=100000, r_heads=6, r_kv=2, r_dim=34, r_vdim=9, r_conv=2,
                            left_scale=-0.5, right_scale=2.0, mlp=ff(9, 4.0)),
                   mamba1(inner=40, state=70, dt_rank=3, conv=2, mlp=ff(20, 1.0))],
                  width=45, vocab=77, emb_scale=0.5, cap=3.0, side=5)


def lively(tensors: Dict[str, torch.Tensor], seed: int = 1) -> None:
    """Make the random weights show more: larger matrices inside the mixers (scores of order one, gates and decays away
    from their middle), positive distance coefficients of order one, a mixing matrix near the identity plus noise, state
    decays spread over a decade, norm weights that differ."""
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        def fill(lo, hi):
            t.copy_((torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype))
        if name.endswith((".left.q", ".left.k", ".left.v", ".right.q", ".right.k", ".right.v", ".right.g", ".mix.in", ".mix.x")):
            t.mul_(8.0)
        elif name.endswith((".right.b", ".right.a", ".mix.dt", ".side.gate", ".side.proj")):
            t.mul_(20.0)
        elif name.endswith((".mlp.gate", ".mlp.up")):
            t.mul_(12.0)
        elif name.endswith((".r1", ".r2")):
            fill(0.2, 1.5)
        elif name.endswith(".talk"):
            t.copy_((torch.eye(t.shape[0]) + 0.4 * torch.randn(t.shape, generator=g)).to(t.dtype))
        elif name.endswith(".mix.A_log"):
            fill(-1.5, 1.0)
        elif name.endswith(".right.A_log"):
            fill(-3.0, 0.0)
        elif name.endswith((".dt_bias", ".dt.b")):
            fill(-3.0, 0.5)
        elif name.endswith((".mix.D", ".right.norm", ".side.norm")):
            fill(0.5, 2.0)
        elif name.endswith(("norm1", "norm2", "final.norm")):
            fill(-0.5, 0.8)
        elif name.endswith(".b") and t.dim() == 1:
            t.mul_(10.0)


def plain_logits(folder: str, requests: Dict[str, List[int]], rounded: bool = False) -> Dict[str, torch.Tensor]:
    cfg, w = read_folder(folder)
    store = P.round_to_bfloat16 if rounded else P._keep
    return {rid: P.forward(cfg, w, toks, store=store) for rid, toks in requests.items()}
