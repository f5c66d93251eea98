"""Bamipel without a GPU: reading config.json, layers that borrow another layer's tensors, tensor names, what the
mixers ask of the cache manager, pages that a sliding window lets go, and the plain implementation's own consistency."""
import numpy as np
import pytest

import bamipel_util as bu
import plain_bamipel as plain


def test_config_reads_every_size_and_refuses_what_it_does_not_know():
    from hfee_b200.config import ConfigError, resolve
    arch, cfg = resolve(bu.BAM_A)
    assert arch.name == "Bamipel" and cfg.width == 64 and cfg.vocab == 200 and cfg.eps == 1e-5
    assert [l.type for l in cfg.layers] == ["delta", "latent_attention", "attention", "latent_attention", "delta"]
    assert [l.weights_of for l in cfg.layers] == [None, None, None, 1, 0]
    assert cfg.layers[0].mixer.taps == 3 and cfg.layers[1].mixer.window == 10 and cfg.layers[2].mixer.window is None
    assert cfg.layers[2].mlp is None and cfg.layers[1].mlp.ff == 80 and cfg.layers[2].mixer.rot.scaling.factor == 8.0
    assert cfg.layers[2].mixer.rot.scaling.original_max_position_embeddings == 64 and cfg.layers[1].mixer.rot.scaling is None
    with pytest.raises(ConfigError, match="not a mixer"):
        resolve(dict(bu.BAM_A, layers=[{"type": "mamba", "mixer": {}, "mlp": None}]))
    with pytest.raises(ConfigError, match="norm"):
        resolve({k: v for k, v in bu.BAM_A.items() if k != "norm"})
    with pytest.raises(ConfigError, match="multiple of kv_heads"):
        resolve(bu.config(32, 50, [bu.delta(3, 2, 8, 8, 2)]))
    with pytest.raises(ConfigError, match="rot_dim"):
        bad = bu.latent(2, 8, 8, 8, 8, 8, None, 10.0, 1.0)
        bad["mixer"]["rot"]["dims"] = 4
        resolve(bu.config(32, 50, [bad]))
    with pytest.raises(ConfigError, match="dense"):
        resolve(bu.config(32, 50, [dict(bu.delta(1, 1, 8, 8, 2), mlp={"kind": "experts", "ff": 8})]))
    layers = [bu.delta(1, 1, 8, 8, 2), bu.delta(1, 1, 8, 8, 2)]
    with pytest.raises(ConfigError, match="not a layer"):
        resolve(bu.config(32, 50, [layers[0], dict(layers[1], weights_of=5)]))
    with pytest.raises(ConfigError, match="another layer"):
        resolve(bu.config(32, 50, [layers[0], dict(bu.delta(1, 1, 8, 16, 2), weights_of=0)]))
    with pytest.raises(ConfigError, match="no tensors of its own"):
        resolve(bu.config(32, 50, [layers[0], dict(layers[0], weights_of=0), dict(layers[0], weights_of=1)]))


def test_layout_names_schedule_and_cache_needs():
    from hfee_b200 import CacheBundle, FixedState, PagedKV
    from hfee_b200.config import resolve
    from hfee_b200.config.spec import RunSpec
    from hfee_b200.parts.model import model_tensor_needs
    arch, cfg = resolve(bu.BAM_B)
    spec = arch.build_spec(cfg)
    # four layers own tensors; the third entry runs the fourth's with cache 2
    assert len(spec.layers) == 4
    assert spec.schedule == (RunSpec(0, 0), RunSpec(1, 1), RunSpec(2, 2), RunSpec(2, 3), RunSpec(3, 4))
    needs = model_tensor_needs(spec)
    assert not any(n.startswith("l2.") for n in needs)
    assert needs["l3.mix.dq"].shape == (16, 96) and needs["l3.mix.dq.norm"].shape == (16,)
    assert needs["l3.mix.uq"].shape == (2 * (24 + 16), 16) and needs["l3.mix.dkv"].shape == (48 + 16, 96)
    assert needs["l3.mix.uk"].shape == (48, 48) and needs["l3.mix.uv"].shape == (16, 48) and needs["l3.mix.g"].shape == (2, 96)
    assert needs["l1.mix.q.conv"].shape == (80, 2) and needs["l1.mix.v.conv"].shape == (40, 2) and needs["l1.mix.norm"].shape == (20,)
    assert needs["l1.mix.A_log"].shape == (2,) and needs["l1.mix.b"].shape == (2, 96) and "l1.mlp.up" not in needs
    assert needs["l4.mix.k"].shape == (64, 96) and needs["l4.mix.g"].shape == (2, 96) and needs["l4.norm2b"].shape == (96,)
    assert needs["l0.mlp.up"].shape == (128, 96) and "l0.mlp.gate" not in needs and needs["head"].shape == (310, 96)
    # what the mixers ask of the cache manager, built without a device
    arch_a, cfg_a = resolve(bu.BAM_A)
    mixers = [layer.parts["mixer"][1] for layer in arch_a.build_spec(cfg_a).layers]
    assert mixers[1].kind == "latent_attention" and mixers[1].kv_rank + mixers[1].rope_dim == 32 and mixers[1].window == 10
    assert mixers[2].kind == "gated_attention" and (mixers[2].head_dim, mixers[2].value_dim) == (32, 16)
    assert PagedKV(1, 32, 10, None, 0) != PagedKV(1, 32, 10) and PagedKV(2, 32, None, None, 16).value_dim == 16
    assert CacheBundle.of(None, conv=FixedState((2, 112)), recurrent=FixedState((4, 16, 24))).state_map()["conv"].shape == (2, 112)


def test_value_pools_of_their_own_size_and_pages_behind_a_window_are_given_back():
    import torch
    from hfee_b200 import CacheBundle, CacheManager, FixedState, PagedKV
    needs = {0: PagedKV(1, 32, 10, None, 0),                       # a latent: nothing cached beside the keys
             1: PagedKV(2, 32, None, None, 16),                    # values of half the keys' size
             2: CacheBundle.of(None, conv=FixedState((2, 12)), recurrent=FixedState((2, 4, 6))),
             3: PagedKV(1, 32, 10, None, 0)}
    m = CacheManager(needs, page_size=16, num_pages=8, max_requests=2, max_context=128, dtype=torch.float32)
    v0, v1, v2, v3 = (m.view(i) for i in range(4))
    assert v0.k.shape == (8, 1, 16, 32) and v0.v is None and v3.v is None and v0.k.data_ptr() != v3.k.data_ptr()
    assert v1.k.shape == (8, 2, 16, 32) and v1.v.shape == (8, 2, 16, 16)
    assert v2.states["conv"].shape == (2, 2, 12) and v2.states["recurrent"].shape == (2, 2, 4, 6)
    assert m.cache_bytes() == 4 * (2 * 8 * 16 * 32 + 8 * 2 * 16 * 48 + 2 * (24 + 48))
    s = m.open()
    v2.states["recurrent"][s].fill_(3.0)
    m.reserve(s, 40); m.commit(s, 40)          # the next token, 40, reads 31..40: page 0 of the windowed group is free
    windowed = [g for g in m.paged if g.need.window == 10][0]
    full = [g for g in m.paged if g.need.window is None][0]
    assert windowed.table[s, 0] == -1 and windowed.first_live[s] == 1 and full.first_live[s] == 0
    m.reserve(s, 58); m.commit(s, 58)          # token 58 reads 49..58: pages 0, 1 and 2 are behind the window
    assert windowed.first_live[s] == 3 and windowed.pool.free_pages == 8 - 1 and full.pool.free_pages == 8 - 4
    m.check_invariants()
    m.close(s)
    assert m.open() == s and float(v2.states["recurrent"][s].abs().max()) == 0 and m.free_pages() == 8


def _random_weights(cfg, seed):
    from hfee_b200.config import resolve
    from hfee_b200.parts.model import model_tensor_needs
    arch, typed = resolve(cfg)
    rng = np.random.default_rng(seed)
    w = {}
    for name, need in model_tensor_needs(arch.build_spec(typed)).items():
        w[name] = rng.normal(size=need.shape) * 0.3 + (1.0 if need.role == "scale" else 0.0)
    return w


def test_plain_implementation_is_causal_and_windows_cut():
    """The oracle itself: a later token changes no earlier logits; a key outside the window of a latent layer has no
    effect on it; a borrowed layer is the same function with another history."""
    cfg = bu.config(16, 30, [bu.latent(2, 8, 4, 6, 8, 10, window=3, base=10.0, scale=0.5)])
    w = _random_weights(cfg, 0)
    a = [3, 7, 1, 9, 4, 4, 2, 8, 5]
    b = list(a); b[2] = 11
    la, lb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    assert np.allclose(la[:2], lb[:2]) and not np.allclose(la[2], lb[2]) and not np.allclose(la[4], lb[4])
    assert np.allclose(la[5:], lb[5:])         # position 5 sees 3, 4, 5 only
    layer = bu.delta(2, 1, 8, 6, 3)
    two = bu.config(16, 30, [layer, dict(layer, weights_of=0)])
    w2 = _random_weights(two, 1)
    own = {**w2, **{k.replace("l0.", "l1."): v for k, v in w2.items() if k.startswith("l0.")}}
    assert np.allclose(plain.forward(two, w2, a), plain.forward(bu.config(16, 30, [layer, layer]), own, a))


def test_plain_delta_rule_recurrence_against_its_closed_form():
    """With g = 1 and beta = 1 a write of an orthonormal key replaces what the state held for it: reading with the same key
    returns the value written last."""
    rng = np.random.default_rng(2)
    k = np.eye(4)[[0, 1, 0, 2]][:, None, :]
    v = rng.normal(size=(4, 1, 3))
    o = plain.delta_rule(k.copy(), k, v, np.ones((4, 1)), np.ones((4, 1)))
    assert np.allclose(o[:, 0], v[:, 0])
    o = plain.delta_rule(k[[0, 0, 0, 0]], k, v, np.ones((4, 1)), np.full((4, 1), 0.5))
    assert np.allclose(o[3, 0], 0.5 * v[2, 0])          # written at 2, halved once more at 3; key 2 is orthogonal
    conv = plain.causal_conv(np.arange(5.0)[:, None], np.array([[1.0, 10.0, 100.0]]))
    assert conv[:, 0].tolist() == [0.0, 100.0, 210.0, 321.0, 432.0]


def test_rotation_frequencies_blend_between_the_two_wavelengths():
    f = plain.frequencies(bu.rot(8, 100.0))
    assert np.allclose(f, [1.0, 100 ** -0.25, 0.1, 100 ** -0.75])
    g = plain.frequencies(bu.rot(8, 100.0, scaling=(4.0, 1.0, 4.0, 64)))      # wavelengths 6.3, 19.9, 62.8, 198.7
    assert np.isclose(g[0], f[0]) and np.isclose(g[3], f[3] / 4.0) and f[1] / 4.0 < g[1] < f[1] and f[2] / 4.0 < g[2] < f[2]
    from hfee_b200.config import RopeScaling
    from hfee_b200.parts.rotary import inverse_frequencies
    assert np.allclose(inverse_frequencies(8, 100.0, RopeScaling(4.0, 1.0, 4.0, 64)), g)


def test_command_line_creates_and_shows_a_model_folder(tmp_path, capsys):
    import json
    from hfee_b200 import cli
    from hfee_b200.config import resolve_model_dir
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights import Checkpoint
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(bu.BAM_B))
    model = tmp_path / "model"
    assert cli.main(["create", str(model), str(cfg_path), "--seed", "2"]) == 0
    arch, cfg = resolve_model_dir(str(model))
    assert arch.name == "Bamipel" and cfg.layers[2].weights_of == 3
    needs = model_tensor_needs(arch.build_spec(cfg))
    Checkpoint(str(model)).check(needs)                 # everything asked for is there, nothing else
    c, w = plain.load(str(model))                       # and the plain reader finds every tensor it wants
    assert plain.forward(c, w, [1, 2, 3]).shape == (3, 310)
    capsys.readouterr()
    assert cli.main(["show", str(model)]) == 0
    out = capsys.readouterr().out
    assert "Bamipel" in out and f"{sum(int(np.prod(n.shape)) for n in needs.values()):,}" in out
