"""The kernels behind the Dobelix parts, each against a few lines of plain float64 arithmetic."""
import numpy as np
import pytest
import torch

import plain_dobelix as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_step(counts, lengths=None, slots=None, max_requests=8):
    """A step of ``counts[i]`` new tokens for request i (slot ``slots[i]``, ``lengths[i]`` tokens cached before)."""
    from hfee_b200.engine.batch import Step, StepBuffers, StepEntry
    slots = list(slots or range(len(counts)))
    held = [0] * max_requests
    for s, n in zip(slots, lengths or [0] * len(counts)):
        held[s] = n
    buffers = StepBuffers(max(64, sum(counts)), max_requests, DEV)
    return Step([StepEntry(s, [0] * c, []) for s, c in zip(slots, counts)], held, buffers)


@pytest.mark.parametrize("taps,width", [(1, 40), (2, 64), (3, 200), (8, 33)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_short_conv_continues_across_portions(taps, width, out_dtype):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(taps)
    w = rng.normal(size=(width, taps))
    seqs = [rng.normal(size=(n, width)) for n in (50, 1, 19)]
    want = [x + plain.causal_conv(x, w) for x in seqs]
    state = torch.full((4, max(taps - 1, 0), width), 7.0, device=DEV)      # stale content of an earlier request
    slots = [2, 0, 3]
    for s in slots:
        state[s].zero_()                                                    # what admission does
    wd = torch.tensor(w, dtype=torch.float32, device=DEV)
    got = [[] for _ in seqs]
    at = [0, 0, 0]
    for sizes in ([17, 1, 2], [1, 0, 16], [2, 0, 1], [30, 0, 0]):          # portions longer and shorter than the history
        live = [i for i, n in enumerate(sizes) if n]
        x = torch.tensor(np.concatenate([seqs[i][at[i]:at[i] + sizes[i]] for i in live]), dtype=torch.float32, device=DEV)
        step = make_step([sizes[i] for i in live], slots=[slots[i] for i in live])
        out = torch.empty(x.shape, dtype=out_dtype, device=DEV)
        ops.short_conv(x, wd, state, step, out)
        o = out.float().cpu().numpy()
        k = 0
        for i in live:
            got[i].append(o[k:k + sizes[i]]); k += sizes[i]; at[i] += sizes[i]
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    for g, r in zip(got, want):
        g = np.concatenate(g)
        assert np.max(np.abs(g - r[:len(g)])) < tol * np.max(np.abs(r))
    assert torch.all(state[1] == 7.0)                                        # a slot not in the batch is untouched


def plain_linear_attention(q, k, v, decay, S):
    """Token by token: S <- decay S + k v^T, o = S^T q.  q, k [T, H, D], v [T, H, V], S [H, D, V]."""
    S = S.copy()
    o = np.zeros(v.shape)
    for t in range(q.shape[0]):
        for h in range(q.shape[1]):
            S[h] = decay[h] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 16), (3, 40, 72), (1, 144, 24), (2, 64, 128)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunked", [False, True, "cuda_cores"])
def test_linear_attention_kernels(heads, dim, vdim, dtype, chunked):
    """Both kernels against the recurrence, over several steps that continue the state; slots out of order."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(heads * dim + vdim)
    decay = np.array([1.0, 0.0, 0.93][:heads])
    lens, slots = [70, 33, 1], [3, 1, 2]
    cols = 2 * heads * dim + heads * vdim
    proj = [torch.tensor(rng.normal(size=(n, cols)) * 0.7, dtype=dtype, device=DEV) for n in lens]
    state = torch.zeros((4, heads, dim, vdim), device=DEV)
    state[0].fill_(3.0)
    ref_state = [np.zeros((heads, dim, vdim)) for _ in lens]
    decay_d = torch.tensor(decay, dtype=torch.float32, device=DEV)
    at = [0, 0, 0]
    ws = torch.empty(ops.linear_attention_workspace(4, 128, heads, dim, vdim), dtype=torch.float32, device=DEV)
    for sizes in ([33, 2, 1], [1, 31, 0], [36, 0, 0]):
        live = [i for i, n in enumerate(sizes) if n]
        x = torch.cat([proj[i][at[i]:at[i] + sizes[i]] for i in live])
        step = make_step([sizes[i] for i in live], slots=[slots[i] for i in live])
        q, k, v = x[:, :heads * dim], x[:, heads * dim:2 * heads * dim], x[:, 2 * heads * dim:]
        out = torch.empty((x.shape[0], heads * vdim), dtype=torch.float32, device=DEV)
        ops.linear_attention(q, k, v, decay_d, state, step, out, heads, dim, vdim, "silu", True, ws, chunked=bool(chunked),
                             tensor_cores=chunked is True)
        o = out.cpu().numpy()
        row = 0
        for i in live:
            n = sizes[i]
            xs = plain.silu(proj[i][at[i]:at[i] + n].double().cpu().numpy())
            if chunked is True and dtype == torch.bfloat16 and dim % 16 == 0:
                # the tensor-core kernels take q, k and v as the bfloat16 values of their activations
                xs = torch.tensor(xs).to(torch.bfloat16).double().numpy()
            want, ref_state[i] = plain_linear_attention(xs[:, :heads * dim].reshape(n, heads, dim),
                                                        xs[:, heads * dim:2 * heads * dim].reshape(n, heads, dim),
                                                        xs[:, 2 * heads * dim:].reshape(n, heads, vdim), decay, ref_state[i])
            assert np.max(np.abs(o[row:row + n] - want.reshape(n, -1))) < 2e-5 * max(1.0, np.max(np.abs(want)))
            row += n
            at[i] += n
    for i, s in enumerate(slots):
        assert np.max(np.abs(state[s].cpu().numpy() - ref_state[i])) < 2e-5 * max(1.0, np.max(np.abs(ref_state[i])))
    assert torch.all(state[0] == 3.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_kernels(dtype):
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(0)
    n, width, inner = 19, 136, 72
    y = rng.normal(size=(n, width)) * 3
    w = 1 + rng.normal(size=width) * 0.3
    res = rng.normal(size=(n, width))
    res_d = torch.tensor(res, dtype=torch.float32, device=DEV)
    ops.rmsnorm_add(torch.tensor(y, dtype=torch.float32, device=DEV), torch.tensor(w, dtype=torch.float32, device=DEV), res_d, 1e-3)
    assert np.max(np.abs(res_d.cpu().numpy() - (res + plain.rms_norm(y, w, 1e-3)))) < 1e-5

    for wide in (136, 2048, 4102, 6144, 9000):        # the 16-byte variants (2 and 8 pieces a thread) and the plain kernel
        yw, ww, rw = rng.normal(size=(5, wide)), 1 + rng.normal(size=wide) * 0.3, rng.normal(size=(5, wide))
        r_d = torch.tensor(rw, dtype=torch.float32, device=DEV)
        cast = torch.empty((5, wide), dtype=dtype, device=DEV)
        ops.rmsnorm_add(torch.tensor(yw, dtype=torch.float32, device=DEV), torch.tensor(ww, dtype=torch.float32, device=DEV),
                        r_d, 1e-3, cast_out=cast)
        assert np.max(np.abs(r_d.cpu().numpy() - (rw + plain.rms_norm(yw, ww, 1e-3)))) < 2e-5
        assert torch.equal(cast, r_d.to(dtype))

    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for wide in (2048, 4096, 4098):                   # 16-byte variants and the plain kernel; the gate a column slice
        xw, ww = rng.normal(size=(3, wide)) * 2, 1 + rng.normal(size=wide) * 0.3
        both = torch.tensor(rng.normal(size=(3, 2 * wide)), dtype=dtype, device=DEV)
        gw, ow = both[:, wide:], torch.empty((3, wide), dtype=dtype, device=DEV)
        ops.norm_gate(torch.tensor(xw, dtype=torch.float32, device=DEV), torch.tensor(ww, dtype=torch.float32, device=DEV), 1e-3, gw, ow)
        want = plain.rms_norm(xw, ww, 1e-3) * plain.sigmoid(gw.double().cpu().numpy())
        assert np.max(np.abs(ow.double().cpu().numpy() - want)) < tol * np.max(np.abs(want))

    g = torch.tensor(rng.normal(size=(n, width)), dtype=dtype, device=DEV)
    out = torch.empty((n, width), dtype=dtype, device=DEV)
    for weight in (torch.tensor(w, dtype=torch.float32, device=DEV), None):
        ops.norm_gate(torch.tensor(y, dtype=torch.float32, device=DEV), weight, 1e-3, g, out)
        want = (plain.rms_norm(y, w, 1e-3) if weight is not None else y) * plain.sigmoid(g.double().cpu().numpy())
        assert np.max(np.abs(out.double().cpu().numpy() - want)) < tol * np.max(np.abs(want))

    gu = torch.tensor(rng.normal(size=(n, 2 * inner)) * 2, dtype=dtype, device=DEV)
    h = torch.empty((n, inner), dtype=dtype, device=DEV)
    gun = gu.double().cpu().numpy()
    for act, fn in (("gelu_tanh", plain.gelu_tanh), ("silu", plain.silu)):
        for granule in (inner, 4):
            ops.gated_act(gu, h, act, granule)
            grp = gun.reshape(n, inner // granule, 2, granule)
            want = (fn(grp[:, :, 0]) * grp[:, :, 1]).reshape(n, inner)
            assert np.max(np.abs(h.double().cpu().numpy() - want)) < tol * np.max(np.abs(want))

    x = torch.tensor(y, dtype=torch.float32, device=DEV)
    ops.scale_(x, 0.37)
    assert np.max(np.abs(x.cpu().numpy() - y * 0.37)) < 1e-5
    c = torch.empty((n, width), dtype=dtype, device=DEV)
    ops.cast_rows(x, c)
    assert torch.equal(c, x.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,hd,rope_dim,chunk", [(4, 2, 16, 8, 5), (3, 1, 40, 40, 16), (2, 2, 24, 0, 0),
                                                              (8, 2, 32, 32, 13), (4, 4, 64, 16, 70), (16, 1, 48, 48, 9)])
@pytest.mark.parametrize("kernel", ["cuda_cores", "chosen"])
def test_qk_norm_rope_and_sigmoid_attention(dtype, heads, kv_heads, hd, rope_dim, chunk, kernel):
    """Norm over the whole projection, rotation of the leading dimensions, values = keys as projected, pages in
    scrambled order, sigmoid weights inside chunks, output gate; two requests, the second continuing its cache."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(hd)
    page, pages = 8, 16
    q_cols, k_cols = heads * hd, kv_heads * hd
    eps, scale, base = 1e-4, 0.3, 77.0
    wq, wk = 1 + 0.3 * rng.normal(size=q_cols), 1 + 0.3 * rng.normal(size=k_cols)
    temp, bias = 1 + 0.3 * rng.normal(size=heads), rng.normal(size=heads)
    lens = [21, 30]
    rows = [torch.tensor(rng.normal(size=(n, q_cols + k_cols)), dtype=dtype, device=DEV) for n in lens]
    gates = [torch.tensor(rng.normal(size=(n, q_cols)), dtype=dtype, device=DEV) for n in lens]
    k_pool = torch.full((pages, kv_heads, page, hd), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((pages, kv_heads, page, hd), float("nan"), dtype=dtype, device=DEV)
    table = torch.full((4, 4), -1, dtype=torch.int32, device=DEV)
    table[1, :3] = torch.tensor([9, 2, 14], dtype=torch.int32)
    table[3, :4] = torch.tensor([5, 0, 11, 3], dtype=torch.int32)
    f32 = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    inv = torch.tensor([base ** (-2.0 * i / rope_dim) for i in range(rope_dim // 2)], dtype=torch.float64, device=DEV)
    got = [[], []]
    for sizes, before in (([21, 13], [0, 0]), ([0, 17], [21, 13])):
        live = [i for i, n in enumerate(sizes) if n]
        step = make_step([sizes[i] for i in live], lengths=[before[i] for i in live], slots=[[1, 3][i] for i in live], max_requests=4)
        x = torch.cat([rows[i][before[i]:before[i] + sizes[i]] for i in live])
        g = torch.cat([gates[i][before[i]:before[i] + sizes[i]] for i in live])
        cs = None
        if rope_dim:
            cs = torch.empty((step.n, rope_dim // 2, 2), dtype=torch.float32, device=DEV)
            ops.rope_table(step.positions, inv, cs)
        q = torch.empty((step.n, q_cols), dtype=dtype, device=DEV)
        ops.qk_norm_rope_cache(x, f32(wq), f32(wk), eps, cs, rope_dim, step.positions, step.slot_of_token, q, k_pool, v_pool,
                               table, page, heads, kv_heads, hd)
        out = torch.empty_like(q)
        if kernel == "chosen":       # the tensor-core kernel where it takes the sizes
            ops.sigmoid_attention(q, k_pool, v_pool, table, page, step, out, heads, kv_heads, hd, scale, 0, chunk,
                                  f32(temp), f32(bias), g)
        else:
            ops.attention_simt_masked(q, k_pool, v_pool, table, page, step.positions, step.slot_of_token, out, heads,
                                      kv_heads, hd, scale, 0, chunk, ops.WEIGHTS_SIGMOID, f32(temp), f32(bias), g)
        o = out.double().cpu().numpy()
        at = 0
        for i in live:
            got[i].append(o[at:at + sizes[i]]); at += sizes[i]
    for i, n in enumerate(lens):
        x = rows[i].double().cpu().numpy()
        qn = plain.rms_norm(x[:, :q_cols], wq, eps).reshape(n, heads, hd)
        kn = plain.rms_norm(x[:, q_cols:], wk, eps).reshape(n, kv_heads, hd)
        v = x[:, q_cols:].reshape(n, kv_heads, hd)
        if rope_dim:
            pos = np.arange(n, dtype=np.float64)
            qn, kn = plain.rotate_half(qn, pos, rope_dim, base), plain.rotate_half(kn, pos, rope_dim, base)
        want = np.zeros((n, heads, hd))
        for h in range(heads):
            kv = h // (heads // kv_heads)
            for t in range(n):
                lo = (t // chunk) * chunk if chunk else 0
                for j in range(lo, t + 1):
                    want[t, h] += plain.sigmoid(float(qn[t, h] @ kn[j, kv]) * scale * temp[h] + bias[h]) * v[j, kv]
        want = want.reshape(n, -1) * plain.sigmoid(gates[i].double().cpu().numpy())
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        assert np.max(np.abs(np.concatenate(got[i]) - want)) < tol * np.max(np.abs(want))


@pytest.mark.parametrize("m,inner", [(1, 512), (7, 512), (16, 512), (40, 512), (300, 512), (1100, 6144)])
@pytest.mark.parametrize("activation", ["gelu_tanh", "silu"])
def test_gated_activation_in_the_product_epilogue(m, inner, activation):
    """act(x W_gate^T) * (x W_up^T) with the activation applied by the product's epilogue, for the row counts
    of every product kernel (the last case: pairs of CTAs on tiles of 256 x 256)."""
    from hfee_b200.kernels import ops
    rng = np.random.default_rng(m)
    k, granule = 256, ops.SWIGLU_GRANULE
    x = torch.tensor(rng.normal(size=(m, k)), dtype=torch.bfloat16, device=DEV)
    gate = torch.tensor(rng.normal(size=(inner, k)) / 16, dtype=torch.bfloat16, device=DEV)
    up = torch.tensor(rng.normal(size=(inner, k)) / 16, dtype=torch.bfloat16, device=DEV)
    w = torch.stack([gate.reshape(inner // granule, granule, k), up.reshape(inner // granule, granule, k)], dim=1)
    w = w.reshape(2 * inner, k).contiguous()
    out = torch.empty((m, inner), dtype=torch.bfloat16, device=DEV)
    scratch = torch.empty((m, 2 * inner), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(x, w, out, granule, scratch, activation)
    xd = x.double().cpu().numpy()
    fn = plain.gelu_tanh if activation == "gelu_tanh" else plain.silu
    want = fn(xd @ gate.double().cpu().numpy().T) * (xd @ up.double().cpu().numpy().T)
    assert np.max(np.abs(out.double().cpu().numpy() - want)) < 1e-2 * np.max(np.abs(want))
    ops.check_status()
