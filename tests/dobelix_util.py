"""Small Dobelix configurations and helpers shared by the Dobelix tests."""
import json
import os

import numpy as np
import torch


def lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def attention(heads, kv_heads, dim, chunk, rot_dims, base, scale, ff=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk},
                      "rot": {"dims": rot_dims, "base": base}, "scale": scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(width, vocab, layers, taps=3, eps=1e-5, embedding_scale=1.0, logit_scale=1.0):
    return {"architecture": "Dobelix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "canon": {"taps": taps}, "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale}


# Two configurations that differ from each other in every size and option.
DOB_A = config(64, 200, [lightning(2, 16, 32, (0.9, 1.0), ff=96),
                         attention(4, 2, 32, chunk=24, rot_dims=16, base=1000.0, scale=0.2),
                         lightning(3, 32, 16, (0.0, 0.5, 0.97), ff=80)],
               taps=3, eps=1e-5, embedding_scale=0.7, logit_scale=1.5)
DOB_B = config(96, 310, [attention(6, 3, 16, chunk=16, rot_dims=16, base=50.0, scale=0.25, ff=128),
                         lightning(1, 80, 72, (0.995,)),
                         attention(2, 2, 48, chunk=100, rot_dims=8, base=2.0e5, scale=0.11, ff=100)],
               taps=4, eps=1e-6, embedding_scale=1.0, logit_scale=1.0)
STD = 0.15


def write_model(path, cfg, seed, dtype="bfloat16", edit=None):
    """A model folder with random weights (stored in ``dtype``); ``edit(tensors)`` may change them first."""
    from hfee_b200.config.registry import resolve
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights.random_init import random_tensors
    from hfee_b200.weights.safetensors_io import write_file
    arch, typed = resolve(cfg)
    needs = model_tensor_needs(arch.build_spec(typed))
    tensors = random_tensors(needs, seed, torch.float32, STD)
    if edit is not None:
        edit(tensors)
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: v.to(store).contiguous() for k, v in tensors.items()})
    return path


def sequences(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


def make_runner(model_dir, dtype, max_tokens, page_size=16, max_requests=4, batch=None, graphs=False, context=None):
    from hfee_b200 import EngineConfig, ModelRunner
    e = EngineConfig(dtype=dtype, page_size=page_size, max_requests=max_requests, max_context=context or max_tokens,
                     max_cache_tokens=max_tokens, max_batch_tokens=batch or max_tokens, use_cuda_graphs=graphs)
    return ModelRunner(model_dir, e)
