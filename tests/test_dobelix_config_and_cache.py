"""Dobelix without a GPU: reading config.json, the layout as parts, tensor names, the cache bundle,
pages that a chunked mask lets go, and the plain implementation's own consistency."""
import numpy as np
import pytest

import dobelix_util as du
import plain_dobelix as plain


def test_config_reads_every_size_and_refuses_what_it_does_not_know():
    from hfee_b200.config import ConfigError, resolve
    arch, cfg = resolve(du.DOB_A)
    assert arch.name == "Dobelix" and cfg.width == 64 and cfg.taps == 3 and cfg.logit_scale == 1.5
    assert [l.type for l in cfg.layers] == ["lightning", "attention", "lightning"]
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 96 and cfg.layers[1].mixer.chunk == 24
    assert cfg.layers[2].mixer.decay == (0.0, 0.5, 0.97)
    bad = dict(du.DOB_A, layers=[{"type": "mamba", "mixer": {}, "mlp": None}])
    with pytest.raises(ConfigError, match="not a mixer"):
        resolve(bad)
    with pytest.raises(ConfigError, match="canon"):
        resolve({k: v for k, v in du.DOB_A.items() if k != "canon"})
    with pytest.raises(ConfigError, match="one number per head"):
        resolve(dict(du.DOB_A, layers=[du.lightning(2, 8, 8, (0.5,))]))
    with pytest.raises(ConfigError, match="dense"):
        resolve(dict(du.DOB_A, layers=[dict(du.lightning(1, 8, 8, (0.5,)), mlp={"kind": "experts", "ff": 8})]))


def test_layout_names_and_cache_needs():
    from hfee_b200 import CacheBundle, FixedState, PagedKV
    from hfee_b200.config import resolve
    from hfee_b200.parts.model import model_tensor_needs
    arch, cfg = resolve(du.DOB_B)
    spec = arch.build_spec(cfg)
    needs = model_tensor_needs(spec)
    assert needs["l0.mix.q.norm"].shape == (96,) and needs["l0.mix.k.norm"].shape == (48,)
    assert needs["l0.mix.pb"].shape == (6,) and needs["l1.canon1"].shape == (96, 4)
    assert "l0.mix.v" not in needs and "l1.mlp.gate" not in needs and "l1.norm2" not in needs
    assert needs["l1.mix.v"].shape == (72, 96) and needs["l1.mix.q"].shape == (80, 96)
    assert needs["head"].shape == (310, 96) and needs["final.norm"].shape == (96,)
    assert spec.layers[0].parts["mixer"][1].chunk == 16 and spec.embedding.scale == 1.0
    # what the layers ask of the cache manager
    assert CacheBundle.of(PagedKV(3, 16, None, 16), conv=FixedState((3, 96))) == \
        CacheBundle(PagedKV(3, 16, None, 16), (("conv", FixedState((3, 96))),))


def test_bundle_views_and_pages_behind_a_chunk_are_given_back():
    import torch
    from hfee_b200 import CacheBundle, CacheManager, FixedState, PagedKV
    needs = {0: CacheBundle.of(PagedKV(1, 8, None, 24), conv=FixedState((2, 16))),
             1: CacheBundle.of(None, conv=FixedState((2, 16)), recurrent=FixedState((2, 4, 4))),
             2: CacheBundle.of(PagedKV(1, 8, None, 24), conv=FixedState((2, 16)))}
    m = CacheManager(needs, page_size=16, num_pages=6, max_requests=2, max_context=96, dtype=torch.float32)
    v0, v1, v2 = m.view(0), m.view(1), m.view(2)
    assert v0.k.shape == (6, 1, 16, 8) and v0.block_table is v2.block_table and v0.k.data_ptr() != v2.k.data_ptr()
    assert v1.k is None and v1.states["recurrent"].shape == (2, 2, 4, 4)
    assert {v.states["conv"].shape for v in (v0, v1, v2)} == {(2, 2, 16)}
    assert len({v.states["conv"].data_ptr() for v in (v0, v1, v2)}) == 3
    s = m.open()
    v1.states["recurrent"][s].fill_(5.0)
    v0.states["conv"][s].fill_(5.0)
    m.reserve(s, 47); m.commit(s, 47)          # the next token, 47, starts reading at 24: page 1; page 0 is free again
    assert m.free_pages() == 6 - 2 and m.paged[0].table[s, 0] == -1
    m.reserve(s, 48); m.commit(s, 48)          # token 48 opens the block 48..71: pages 1 and 2 are behind it
    assert m.free_pages() == 6 and m.paged[0].first_live[s] == 3
    m.reserve(s, 90); m.commit(s, 90)          # block 72..95 lies in pages 4 and 5
    assert m.paged[0].first_live[s] == 4
    m.check_invariants()
    m.close(s)
    s2 = m.open()                               # the same slot again: states are cleared
    assert s2 == s and float(v1.states["recurrent"][s].abs().max()) == 0 and float(v0.states["conv"][s].abs().max()) == 0
    assert m.free_pages() == 6


def test_plain_implementation_is_causal_and_chunks_cut():
    """The oracle itself: a later token changes no earlier logits; a key in another chunk has no effect on
    the attention layer, and lightning with decay 0 sees only the current token."""
    rng = np.random.default_rng(0)
    cfg = du.config(16, 30, [du.attention(2, 1, 8, chunk=4, rot_dims=4, base=10.0, scale=0.5)], taps=1)
    W = {"embed": rng.normal(size=(30, 16)), "final.norm": np.ones(16), "head": rng.normal(size=(30, 16)),
         "l0.norm1": np.ones(16), "l0.canon1": np.zeros((16, 1)), "l0.mix.q": rng.normal(size=(16, 16)),
         "l0.mix.k": rng.normal(size=(8, 16)), "l0.mix.g": rng.normal(size=(16, 16)), "l0.mix.o": rng.normal(size=(16, 16)),
         "l0.mix.q.norm": np.ones(16), "l0.mix.k.norm": np.ones(8), "l0.mix.temp": np.ones(2), "l0.mix.pb": np.zeros(2)}
    a = [3, 7, 1, 9, 4, 4, 2, 8, 5]
    b = list(a); b[3] = 11                     # position 3 is the last of chunk 0
    la, lb = plain.forward(cfg, W, a), plain.forward(cfg, W, b)
    assert np.allclose(la[:3], lb[:3]) and not np.allclose(la[3], lb[3])
    assert np.allclose(la[4:], lb[4:])         # chunk 1 and 2 never see position 3
    h = rng.normal(size=(6, 16))
    Wl = {"q": rng.normal(size=(8, 16)), "k": rng.normal(size=(8, 16)), "v": rng.normal(size=(8, 16)),
          "g": rng.normal(size=(8, 16)), "o": rng.normal(size=(16, 8)), "norm": np.ones(8)}
    m = {"heads": 1, "dim": 8, "vdim": 8, "decay": [0.0]}
    whole = plain.lightning_mixer(h, Wl, "", m, 1e-5)
    alone = np.concatenate([plain.lightning_mixer(h[t:t + 1], Wl, "", m, 1e-5) for t in range(6)])
    assert np.allclose(whole, alone)
    assert np.allclose(plain.gelu_tanh(np.array([0.0, 10.0, -10.0])), [0.0, 10.0, 0.0], atol=1e-6)


def test_command_line_creates_and_shows_a_model_folder(tmp_path, capsys):
    import json
    from hfee_b200 import cli
    from hfee_b200.config import resolve_model_dir
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights import Checkpoint
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(du.DOB_B))
    model = tmp_path / "model"
    assert cli.main(["create", str(model), str(cfg_path), "--seed", "2"]) == 0
    arch, cfg = resolve_model_dir(str(model))
    assert arch.name == "Dobelix" and cfg.taps == 4
    needs = model_tensor_needs(arch.build_spec(cfg))
    Checkpoint(str(model)).check(needs)                 # everything asked for is there, nothing else
    capsys.readouterr()
    assert cli.main(["show", str(model)]) == 0
    out = capsys.readouterr().out
    assert "Dobelix" in out and f"{sum(int(np.prod(n.shape)) for n in needs.values()):,}" in out
