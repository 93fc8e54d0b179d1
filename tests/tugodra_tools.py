"""Small Tugodra configurations, model folders for them and plain logits, for the tests of that design.

The sizes differ from layer to layer and between the configurations and avoid values that hide a fault: value sizes
unlike key sizes (smaller and larger), a rotation of part of a head, head groups of one and of several, windows that
divide neither a page nor a tile, a borrowing layer whose window is wider than its lender's, a lender without a window,
routers with one group, with groups of one expert, with one expert per token, experts without a shared one, a layer
without a feed-forward."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional

import torch

import plain_tugodra as P
from tufirax_tools import read_folder, write_folder      # (folders are written by the framework's random-weights mode)


def moe(ff=24, experts=6, top=2, groups=3, keep=2, shared=16):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router, "shared": None if shared is None else {"ff": shared}}


def attention(heads=6, kv_heads=2, dim=24, vdim=16, window: Optional[int] = 13, rot_dims=None, base=500.0, scale=0.3,
              kv_from: Optional[int] = None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"dims": rot_dims or dim, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": copy.deepcopy(mlp)}


def latent(heads=3, dim=24, rot_dim=16, rot_dims=None, vdim=20, kv_rank=40, base=10000.0, scale=0.17, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"dims": rot_dims or rot_dim, "base": base}},
            "mlp": copy.deepcopy(mlp)}


def mlstm(heads=3, dim=12, vdim=20, cap=8.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": copy.deepcopy(mlp)}


def config(layers: List[dict], width=48, vocab=131, eps=1e-5, scale=5.5) -> dict:
    return {"architecture": "Tugodra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": copy.deepcopy(layers)}


def small_a() -> dict:
    """Every mixer; a value narrower than the key and one wider; part of a head rotated; layer 4 borrows layer 1's keys with
    a wider window, layer 5 borrows from a lender that has no window; one group, groups of one, no shared expert, no
    feed-forward."""
    return config([mlstm(mlp=moe()),
                   attention(mlp=moe(ff=20, experts=4, top=1, groups=None, shared=None)),
                   latent(mlp=moe(ff=16, experts=4, top=3, groups=4, keep=3, shared=24)),
                   attention(heads=4, kv_heads=4, dim=8, vdim=12, window=None, rot_dims=4, base=30.0, scale=0.5, mlp=None),
                   attention(window=29, kv_from=1, scale=0.2, mlp=moe()),
                   attention(heads=4, kv_heads=4, dim=8, vdim=12, window=7, rot_dims=4, base=30.0, scale=0.4, kv_from=3, mlp=moe(top=3)),
                   mlstm(heads=2, dim=20, vdim=8, cap=15.0, mlp=None),
                   latent(heads=2, dim=16, rot_dim=8, vdim=32, kv_rank=24, base=500.0, scale=0.3, mlp=moe(experts=8, top=4, groups=2, keep=1))])


def small_b() -> dict:
    """Sizes the tensor-core kernels are built for: heads of 64 with values of 64 in groups of four, latent rows of
    64 + 32 elements, multiples of 16 everywhere, windows that end inside a page and inside a 64-key tile."""
    return config([attention(heads=8, kv_heads=2, dim=64, vdim=64, window=40, base=1e6, scale=0.19, mlp=moe(ff=32, experts=8, top=3, groups=4, keep=2, shared=48)),
                   mlstm(heads=2, dim=32, vdim=64, cap=12.0, mlp=moe(ff=32, experts=4, top=2, groups=2, keep=2, shared=None)),
                   latent(heads=4, dim=32, rot_dim=32, vdim=48, kv_rank=64, scale=0.11, mlp=moe(ff=48, experts=6, top=2, groups=1, keep=1, shared=32)),
                   attention(heads=8, kv_heads=2, dim=64, vdim=64, window=75, base=1e6, scale=0.12, kv_from=0, mlp=None)],
                  width=64, vocab=203, eps=1e-6, scale=3.0)


def odd_shapes() -> dict:
    """Sizes that no fast path is made for: a width and a vocabulary that are no multiples of 8, odd head and value sizes, one
    head, a window of five keys, a key size above a warp in the matrix memory, groups of one expert."""
    return config([attention(heads=3, kv_heads=3, dim=10, vdim=7, window=5, rot_dims=6, base=7.0, scale=0.4, mlp=moe(ff=9, experts=4, top=2, groups=4, keep=4, shared=5)),
                   mlstm(heads=1, dim=5, vdim=3, cap=6.0, mlp=None),
                   latent(heads=1, dim=9, rot_dim=6, vdim=7, kv_rank=35, scale=0.4, mlp=moe(ff=11, experts=6, top=3, groups=2, keep=1, shared=None)),
                   mlstm(heads=5, dim=40, vdim=9, cap=20.0, mlp=moe(ff=7, experts=3, top=3, groups=1, keep=1, shared=13)),
                   attention(heads=6, kv_heads=2, dim=6, vdim=18, window=33, rot_dims=2, base=3.0, scale=0.25, mlp=None)],
                  width=44, vocab=77, scale=2.0)


def lively(tensors: Dict[str, torch.Tensor], seed: int = 1) -> None:
    """Make the random weights show more: larger matrices inside the mixers (scores of order one, gates away from a half,
    input and forget gates that move over their whole range), routers that decide clearly, corrections that change the
    choice, sinks of order one, norm scalars, weights and biases that differ."""
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        def fill(lo, hi):
            t.copy_((torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype))
        if name.endswith((".mix.q", ".mix.k", ".mix.dkv", ".mix.g")):
            t.mul_(10.0)
        elif name.endswith((".mix.uk", ".mix.uv", ".mix.v")):
            t.mul_(6.0)
        elif name.endswith((".mix.i", ".mix.f")):
            t.mul_(60.0)
        elif name.endswith((".mix.i.b", ".mix.f.b")):
            fill(-2.0, 3.0)
        elif name.endswith(".mix.sink"):
            fill(-2.0, 3.0)
        elif name.endswith(".mlp.router"):
            t.mul_(40.0)
        elif name.endswith(".mlp.correction"):
            fill(-0.4, 0.4)
        elif name.endswith(".mlp.shared.sg"):
            t.mul_(20.0)
        elif name.endswith(".alpha"):
            fill(0.3, 1.4)
        elif name.endswith((".mix.dkv.norm", ".mix.norm", "norm1b", "norm2b")):
            fill(0.5, 2.0)
        elif name.endswith(".b") and "norm" in name:
            fill(-0.3, 0.3)


def plain_logits(folder: str, requests: Dict[str, List[int]], rounded: bool = False) -> Dict[str, torch.Tensor]:
    cfg, w = read_folder(folder)
    store = P.round_to_bfloat16 if rounded else P._keep
    return {rid: P.forward(cfg, w, toks, store=store) for rid, toks in requests.items()}
