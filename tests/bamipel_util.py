"""Small Bamipel configurations and helpers shared by the Bamipel tests."""
import json
import os

import numpy as np
import torch

from dobelix_util import make_runner, sequences  # noqa: F401  (the same engine settings and token draws)


def _mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        factor, low, high, original = scaling
        r["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return r


def attention(heads, kv_heads, dim, vdim, rot_dims, base, scale, scaling=None, ff=None, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot(rot_dims, base, scaling), "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": _mlp(ff)}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base, scale, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": rot(rot_dim, base), "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": _mlp(ff)}


def delta(heads, kv_heads, dim, vdim, taps, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps},
            "mlp": _mlp(ff)}


def again(layers, j):
    """An entry that runs layer j once more with a cache of its own."""
    return dict(layers[j], weights_of=j)


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Bamipel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}


# Two configurations that differ from each other in every size and option.
_A = [delta(4, 2, 16, 24, 3, ff=96),
      latent(3, 16, 8, 24, 40, 24, window=10, base=1000.0, scale=0.2, ff=80),
      attention(4, 2, 32, 16, 16, 500.0, 0.3, scaling=(8.0, 1.0, 4.0, 64))]
BAM_A = config(64, 200, _A + [again(_A, 1), again(_A, 0)], eps=1e-5)
_B = [attention(6, 6, 16, 16, 16, 50.0, 0.25, ff=128),
      delta(2, 2, 40, 20, 2),
      None,                                             # filled below: uses the tensors of a LATER layer
      latent(2, 24, 16, 8, 16, 48, window=100, base=2.0e5, scale=0.11, ff=100),
      attention(2, 1, 64, 64, 32, 3.0e4, 0.125, scaling=(4.0, 1.0, 2.0, 32), ff=72)]
_B[2] = again(_B, 3)
BAM_B = config(96, 310, _B, eps=1e-6)
STD = 0.15


def write_model(path, cfg, seed, dtype="bfloat16", edit=None):
    """A model folder with random weights (stored in ``dtype``); ``edit(tensors)`` may change them first.
    The decay inputs get values that spread the decays over (0, 1) instead of bunching them near 0.5."""
    from hfee_b200.config.registry import resolve
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights.random_init import random_tensors
    from hfee_b200.weights.safetensors_io import write_file
    arch, typed = resolve(cfg)
    needs = model_tensor_needs(arch.build_spec(typed))
    tensors = random_tensors(needs, seed, torch.float32, STD)
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        if name.endswith("mix.A_log"):
            t.copy_(torch.empty(t.shape).uniform_(-4.0, 1.0, generator=g))
        if name.endswith("mix.dt_bias"):
            t.copy_(torch.empty(t.shape).uniform_(-3.0, 1.0, generator=g))
    if edit is not None:
        edit(tensors)
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: v.to(store).contiguous() for k, v in tensors.items()})
    return path


FIRST_A, FIRST_B, LATER = 0, 1, 2        # embedding dimensions that mark the tokens of the far-token tests


def mark_first_tokens(tensors, size=1.0):
    """Tokens 0 and 1 (which the far-token tests put at the start of a sequence only) carry a large entry in a dimension
    of their own, every other token in a third one: after the input norm a projection can pick out "first token A",
    "first token B" and "any later token" by one column of its weight each."""
    emb = tensors["embed"]
    emb[:, [FIRST_A, FIRST_B, LATER]] = 0.0
    emb[0, FIRST_A] = size
    emb[1, FIRST_B] = size
    emb[2:, LATER] = size
