"""Pakarax on the GPU: every mechanism alone against the plain implementation
(`plain_pakarax`), then whole models through the engine under every way of
cutting the work, and generation through the entry point."""

import math

import numpy as np
import pytest
import torch

import pakarax_models as pm
import plain_pakarax as pp
from test_kegasun_gpu import FakeBatch, i32, ops, relerr
from test_kernels_gpu import _paged

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def f32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


# ------------------------------------------------------------- mechanisms
CUTS = ({0: 37, 1: 9, 2: 1}, {0: 1, 2: 2}, {2: 1}, {0: 2, 2: 14}, {2: 15}, {0: 30})  # rows per sequence and step


@pytest.mark.parametrize("C,col0,ld", [(20, 3, 30), (24, 4, 32)])  # one channel a thread; four (every size a multiple of 4)
@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_short_convolution_carried_through_its_state(taps, C, col0, ld):
    """Three sequences of unequal lengths in steps of unequal sizes, down to one
    and two rows (fewer than the filter looks back), in slots that are not in
    order: every step goes on from the inputs the steps before left; a slot
    taken again starts from zeros."""
    g = torch.Generator().manual_seed(taps)
    lens, slots = {0: 70, 1: 9, 2: 33}, {0: 3, 1: 0, 2: 6}
    proj = {s: torch.randn(n, ld, generator=g) for s, n in lens.items()}
    bias, w, cb = torch.randn(C, generator=g), torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    extra = 8  # the state vector holds more than the filter's inputs (another part's floats)
    state = torch.zeros(8, (taps - 1) * C + extra, device=DEV)
    state[:, (taps - 1) * C:] = 5.0
    fed = {s: 0 for s in lens}
    got = {s: [] for s in lens}
    for cuts in CUTS:
        ids = list(cuts)
        b = FakeBatch([[0] * cuts[s] for s in ids], [slots[s] for s in ids], [fed[s] for s in ids])
        rows = torch.cat([proj[s][fed[s]:fed[s] + cuts[s]] for s in ids]).to(DEV)
        out, lo = ops().short_conv(rows, col0, C, bias.to(DEV), w.t().contiguous().to(DEV), cb.to(DEV),
                                   state if taps > 1 else None, b, also_bf16=True)
        assert torch.equal(lo, out.to(torch.bfloat16))
        ops().conv_state_update(rows, col0, C, bias.to(DEV), taps, state, b)
        for j, s in enumerate(ids):
            got[s].append(out[b.row0[j]:b.row0[j + 1]].cpu())
            fed[s] += cuts[s]

    def ref(s):
        u = proj[s][:, col0:col0 + C].double().numpy() + bias.double().numpy()
        return pp.causal_conv(u, w.double().numpy(), cb.double().numpy())

    for s in lens:
        assert fed[s] == lens[s]
        assert relerr(torch.cat(got[s]), ref(s)) < 3e-6, s
    assert bool((state[:, (taps - 1) * C:] == 5.0).all())  # the floats beside the filter's are left alone
    if taps > 1:
        state[0].zero_()
        b = FakeBatch([[0] * 9], [0], [0])
        out = ops().short_conv(proj[1].to(DEV), col0, C, bias.to(DEV), w.t().contiguous().to(DEV), cb.to(DEV), state, b)
        assert relerr(out, ref(1)) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dim,vdim,taps,temp", [(4, 2, 16, 24, 3, (0.3, 7)), (3, 3, 40, 20, 4, (0.5, 64)),
                                                       (6, 1, 8, 8, 1, None), (2, 1, 64, 64, 2, (1.0, 1)),
                                                       (3, 1, 10, 6, 3, (0.3, 5))])  # the last: one element a thread
def test_convolved_q_k_v_temperature_and_cache_write(dtype, nq, nkv, dim, vdim, taps, temp):
    """Two steps of two sequences: q out with its temperature, k and v in the
    paged cache at the rows' positions, heads padded with zeros, the second
    step continuing from the first one's last inputs; positions around the
    temperature's steps and a page's edge."""
    g = torch.Generator().manual_seed(nq + dim)
    pad = (max(dim, vdim) + 15) // 16 * 16
    C = nq * dim + nkv * (dim + vdim)
    starts = {0: 0, 1: 60}  # sequence 1 begins at position 60 with an empty history (its state is zero)
    lens = {0: 15, 1: 9}
    proj = {s: torch.randn(n, C, generator=g) for s, n in lens.items()}
    bias, w = torch.randn(C, generator=g), torch.randn(C, taps, generator=g)
    state = torch.zeros(4, max(1, (taps - 1) * C), device=DEV)
    k_pages = torch.full((6, nkv, 64, pad), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full((6, nkv, 64, pad), float("nan"), dtype=dtype, device=DEV)
    table = i32([[3, 5, 9], [9, 9, 9], [4, 1, 9], [9, 9, 9]])
    slots = {0: 0, 1: 2}
    qs = {0: [], 1: []}
    fed = {0: 0, 1: 0}
    for cuts in ({0: 13, 1: 2}, {0: 2, 1: 7}):
        ids = list(cuts)
        b = FakeBatch([[0] * cuts[s] for s in ids], [slots[s] for s in ids], [starts[s] + fed[s] for s in ids])
        rows = torch.cat([proj[s][fed[s]:fed[s] + cuts[s]] for s in ids]).to(DEV)
        q = ops().conv_qkv_post(rows, bias.to(DEV), w.t().contiguous().to(DEV), state if taps > 1 else None, b, k_pages, v_pages,
                                table, 64, nq, nkv, dim, vdim, pad, temp[0] if temp else 0.0,
                                temp[1] if temp else 1, True, dtype)
        ops().conv_state_update(rows, 0, C, bias.to(DEV), taps, state, b)
        for j, s in enumerate(ids):
            qs[s].append(q[b.row0[j]:b.row0[j + 1]].float().cpu())
            fed[s] += cuts[s]
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for s in (0, 1):
        y = pp.causal_conv(proj[s].double().numpy() + bias.double().numpy(), w.double().numpy())
        pos = starts[s] + np.arange(lens[s])
        qr = y[:, :nq * dim].reshape(-1, nq, dim)
        if temp:
            qr = qr * pp.query_temperature(pos, temp[0], temp[1])[:, None, None]
        got = torch.cat(qs[s]).reshape(-1, nq, pad)
        assert relerr(got[:, :, :dim], qr) < tol
        assert bool((got[:, :, dim:] == 0).all())
        kr = y[:, nq * dim:nq * dim + nkv * dim].reshape(-1, nkv, dim)
        vr = y[:, nq * dim + nkv * dim:].reshape(-1, nkv, vdim)
        for t, p in enumerate(pos):
            page = int(table[slots[s], p // 64])
            assert relerr(k_pages[page, :, p % 64, :dim], kr[t]) < tol
            assert relerr(v_pages[page, :, p % 64, :vdim], vr[t]) < tol
            assert bool((k_pages[page, :, p % 64, dim:] == 0).all())
            assert bool((v_pages[page, :, p % 64, vdim:] == 0).all())


def _slope_ref(q, ks, vs, seqs, scale, window, sink, slopes, dtype):
    outs, r = [], 0
    for (start, n), k, v in zip(seqs, ks, vs):
        kk, vv = k.to(dtype).double().numpy(), v.to(dtype).double().numpy()
        for t in range(n):
            i = start + t
            lo = 0 if not window else max(0, i - window + 1)
            o = np.zeros((q.shape[1], vv.shape[2]))
            for h in range(q.shape[1]):
                kvh = h // (q.shape[1] // kk.shape[1])
                s = (kk[lo:i + 1, kvh] @ q[r + t, h].to(dtype).double().numpy()) * scale
                s = s - slopes[h] * (i - np.arange(lo, i + 1))
                mx = max(s.max(), sink[h])
                e = np.exp(s - mx)
                o[h] = (e[:, None] * vv[lo:i + 1, kvh]).sum(0) / (e.sum() + math.exp(sink[h] - mx))
            outs.append(o)
        r += n
    return np.stack(outs)


SLOPE_CASES = [  # nq, nkv, d, [(start, n_new)], window
    (8, 4, 112, [(0, 70), (130, 3), (0, 1)], None),
    (6, 1, 64, [(0, 129), (63, 2)], None),
    (4, 2, 80, [(0, 40), (100, 30)], 37),
    (3, 3, 40, [(0, 66)], None),
    (16, 1, 128, [(0, 200)], None),
]


@pytest.mark.parametrize("kernel", ["plain_f32", "plain_bf16", "prefill_bf16", "prefill_tc_bf16", "decode_bf16",
                                    "dispatch_bf16"])
@pytest.mark.parametrize("nq,nkv,d,seqs,window", SLOPE_CASES)
def test_attention_with_distance_slopes_and_a_sink_in_every_kernel(kernel, nq, nkv, d, seqs, window):
    """slope * (i - j) comes off every score, beside a sink.  The first key of
    every sequence is made to stand out (its key is a large multiple of the
    mean query), so that a steep head forgets it with distance while a flat one
    still finds it hundreds of tokens later."""
    if not kernel.startswith("plain") and d % 16:
        pytest.skip("multiples of 16")
    if kernel == "prefill_tc_bf16" and d not in (64, 128):
        pytest.skip("head sizes 64 and 128")
    g = torch.Generator().manual_seed(nq + d)
    dtype = torch.float32 if kernel == "plain_f32" else torch.bfloat16
    if kernel == "decode_bf16":
        seqs = [(a + b - 1, 1) for a, b in seqs]
    slots, table, kp, vp, ks, vs = _paged([a + b for a, b in seqs], nkv, d, dtype, g)
    R = sum(b for _, b in seqs)
    q = torch.randn(R, nq, d, generator=g) + 1.0
    scale = d ** -0.5
    # the far key: along the queries' common direction, worth about 12 units of score
    far = torch.ones(d) * (12.0 / (scale * d))
    kd_host = kp.clone()
    for i in range(len(seqs)):
        ks[i][0] = far
        kd_host[int(table[slots[i], 0]), :, 0] = far.to(dtype)
    slopes = np.array([2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq)])
    sink = np.linspace(-3.0, 4.0, nq)
    ref = _slope_ref(q, ks, vs, seqs, scale, window, sink, slopes, dtype)
    flat = _slope_ref(q, ks, vs, seqs, scale, window, sink, np.zeros(nq), dtype)
    assert np.abs(ref - flat).max() > 0.2  # the slopes matter in this case
    sd, ld = f32(sink), f32(slopes)
    qd = q.reshape(R, nq * d).to(dtype).to(DEV)
    kd, vd, td = kd_host.to(DEV), vp.to(DEV), table.to(DEV)
    row_pos = i32([a + j for a, b in seqs for j in range(b)])
    row_slot = i32([slots[i] for i, (a, b) in enumerate(seqs) for _ in range(b)])
    outs = []
    if kernel.startswith("plain"):
        outs.append(ops().attention_plain(qd, kd, vd, td, 64, row_pos, row_slot, nq, nkv, d, window, scale,
                                          sink=sd, slopes=ld))
    elif kernel == "decode_bf16":
        for splits in (1, 2, 3):  # alone, merged inside a cluster, merged by the combine kernel
            outs.append(ops().attention_decode(qd, kd, vd, td, 64, row_pos, row_slot, nq, nkv, d, window, scale,
                                               n_splits=splits, sink=sd, slopes=ld))
    else:
        row0 = [0]
        for _, b in seqs:
            row0.append(row0[-1] + b)
        if kernel == "dispatch_bf16":  # what a model's step calls: picks the kernel itself
            b = FakeBatch([[0] * n for _, n in seqs], slots, [a for a, _ in seqs])
            b.is_decode, b.max_new = False, max(n for _, n in seqs)
            b.max_context = max(a + n for a, n in seqs)
            outs.append(ops().attention(qd, kd, vd, td, 64, b, nq, nkv, d, window, scale, sink=sd, slopes=ld))
        else:
            fn = ops().attention_prefill_tc if kernel == "prefill_tc_bf16" else ops().attention_prefill
            outs.append(fn(qd, kd, vd, td, 64, i32(slots), i32([a for a, _ in seqs]), i32([b for _, b in seqs]),
                           i32(row0), max(b for _, b in seqs), nq, nkv, d, window, scale, sink=sd, slopes=ld))
    ops().check_device_errors(DEV)
    for out in outs:
        assert not bool(torch.isnan(out.float()).any())
        assert relerr(out.reshape(R, nq, d), ref) < (3e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,blocks", [(48, 3), (10, 1), (130, 5), (256, 2)])
def test_gated_recurrence_carried_through_its_state(W, blocks, out_dtype, chunked):
    """The recurrence over sequences cut into unequal steps; S goes on from step
    to step in the state vector, beside the convolution's floats, which it
    leaves alone; gates that swing from shut to open, decays from 2^-8 to 1.
    Both kernels: the row-by-row walk and the one that folds 128 rows at a time
    (whole tiles, partial ones, single rows)."""
    g = torch.Generator().manual_seed(W)
    K = W // blocks
    lens, slots = {0: 335, 1: 9, 2: 33}, {0: 3, 1: 0, 2: 6}
    cuts_list = ({0: 200, 1: 9, 2: 1}, {0: 1, 2: 2}, {2: 1}, {0: 2, 2: 14}, {2: 15}, {0: 132})
    ld, y_off, off = W + 5, 2, 11
    u = {s: torch.randn(n, W, generator=g) for s, n in lens.items()}
    gates = {s: torch.randn(n, 2 * W, generator=g) * 4 for s, n in lens.items()}
    proj = {s: torch.randn(n, ld, generator=g) for s, n in lens.items()}
    rb, ib, yb = (torch.randn(W, generator=g) for _ in range(3))
    lam = torch.randn(W, generator=g) * 3
    state = torch.zeros(8, off + W, device=DEV)
    state[:, :off] = 7.0
    fed = {s: 0 for s in lens}
    got = {s: [] for s in lens}
    for cuts in cuts_list:
        ids = list(cuts)
        b = FakeBatch([[0] * cuts[s] for s in ids], [slots[s] for s in ids], [fed[s] for s in ids])
        cat = lambda d: torch.cat([d[s][fed[s]:fed[s] + cuts[s]] for s in ids]).to(DEV)  # noqa: E731
        out = ops().rglru_scan(cat(u), cat(gates), rb.to(DEV), ib.to(DEV), lam.to(DEV), 8.0, cat(proj), y_off,
                               yb.to(DEV), state, off, b, blocks, out_dtype, max_rows=10 ** 6 if chunked else None)
        for j, s in enumerate(ids):
            got[s].append(out[b.row0[j]:b.row0[j + 1]].float().cpu())
            fed[s] += cuts[s]
    assert bool((state[:, :off] == 7.0).all())
    for s, n in lens.items():
        gs = gates[s].double().numpy().reshape(n, blocks, 2, K)
        r = pp.sigmoid(gs[:, :, 0].reshape(n, W) + rb.double().numpy())
        i = pp.sigmoid(gs[:, :, 1].reshape(n, W) + ib.double().numpy())
        a = np.exp(-8.0 * r * pp.softplus(lam.double().numpy()))
        y = pp.gelu_tanh(proj[s][:, y_off:y_off + W].double().numpy() + yb.double().numpy())
        S, ref = np.zeros(W), []
        for t in range(n):
            S = a[t] * S + np.sqrt(1 - a[t] ** 2) * (i[t] * u[s][t].double().numpy())
            ref.append(S * y[t])
        assert relerr(torch.cat(got[s]), np.stack(ref)) < (5e-6 if out_dtype == torch.float32 else 8e-3), s


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("taps", [2, 4])
def test_the_recurrence_kernel_also_keeps_the_convolutions_last_inputs(chunked, taps):
    """Given the convolution's columns, the recurrence's kernel leaves the same
    last inputs in the state as `conv_state_update` does, for steps shorter and
    longer than the filter."""
    g = torch.Generator().manual_seed(taps)
    W, ld, x_off = 12, 40, 20
    xb = torch.randn(W, generator=g)
    lam = torch.randn(W, generator=g)
    T = taps - 1
    a, b_ = torch.zeros(4, T * W + W, device=DEV), torch.zeros(4, T * W + W, device=DEV)
    for n in (1, 2, 7, 1, 140, 3):
        batch = FakeBatch([[0] * n, [0] * 2], [2, 0], [0, 0])
        R = n + 2
        proj = torch.randn(R, ld, generator=g).to(DEV)
        u, gates = torch.randn(R, W, generator=g).to(DEV), torch.randn(R, 2 * W, generator=g).to(DEV)
        ops().rglru_scan(u, gates, None, None, lam.to(DEV), 8.0, proj, 0, None, a, T * W, batch, 1, torch.float32,
                         max_rows=10 ** 6 if chunked else None, conv_tail=(x_off, xb.to(DEV), taps, 0))
        ops().rglru_scan(u, gates, None, None, lam.to(DEV), 8.0, proj, 0, None, b_, T * W, batch, 1, torch.float32,
                         max_rows=10 ** 6 if chunked else None)
        ops().conv_state_update(proj, x_off, W, xb.to(DEV), taps, b_, batch)
        assert torch.equal(a, b_)
    assert float(a[:, :T * W].abs().max()) > 0


@pytest.mark.parametrize("chunked", [False, True])
def test_a_slow_decay_keeps_its_digits(chunked):
    """a within 1e-6 of one: sqrt(1 - a^2) must not be lost to rounding, and S
    builds up over a thousand steps as the closed form says."""
    W, n = 4, 1200
    lam = torch.full((W,), -16.0)  # softplus = 1.1e-7: log a = -8 r * 1.1e-7
    gates = torch.zeros(n, 2 * W)
    gates[:, :] = 30.0  # r = i = 1
    u = torch.ones(n, W)
    proj = torch.full((n, W), 30.0)  # gelu(30) = 30
    state = torch.zeros(2, W, device=DEV)
    b = FakeBatch([[0] * n], [1], [0])
    out = ops().rglru_scan(u.to(DEV), gates.to(DEV), None, None, lam.to(DEV), 8.0, proj.to(DEV), 0, None, state, 0,
                           b, 1, torch.float32, max_rows=n if chunked else None).cpu().double().numpy()
    la = -8.0 * pp.softplus(np.array(-16.0))
    a = np.exp(la)
    want = 30.0 * np.sqrt(-np.expm1(2 * la)) * (1 - a ** np.arange(1, n + 1)) / (1 - a)
    assert np.abs(out[:, 0] - want).max() / want.max() < 2e-4


def test_two_branches_normed_and_averaged():
    g = torch.Generator().manual_seed(0)
    for R, H in ((1, 64), (5, 100), (70, 1024), (3, 5000), (2, 9000)):  # every form of the kernel
        a, b = torch.randn(R, H, generator=g) * 3, torch.randn(R, H, generator=g) * 0.01
        ab, wa, wb = torch.randn(H, generator=g), torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g)
        ref = 0.5 * (pp.rms_norm(a.double().numpy() + ab.double().numpy(), wa.double().numpy(), 1e-5)
                     + pp.rms_norm(b.double().numpy(), wb.double().numpy(), 1e-5))
        out = ops().branch_norm_mean(a.to(DEV), ab.to(DEV), wa.to(DEV), b.to(DEV), wb.to(DEV), 1e-5)
        assert relerr(out, ref) < 3e-6
        ref = 0.5 * (pp.rms_norm(a.double().numpy(), wa.double().numpy(), 1e-5)
                     + pp.rms_norm(b.double().numpy(), wb.double().numpy(), 1e-5))
        assert relerr(ops().branch_norm_mean(a.to(DEV), None, wa.to(DEV), b.to(DEV), wb.to(DEV), 1e-5), ref) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("alternating", [False, True])
@pytest.mark.parametrize("I", [52, 64])  # one output a thread; eight
def test_clamped_gated_activation(dtype, alternating, I):
    g = torch.Generator().manual_seed(1)
    R, limit = 7, 1.25
    gate, up = (torch.randn(R, I, generator=g) * 3).to(dtype), (torch.randn(R, I, generator=g) * 3).to(dtype)
    gate[0, :4] = torch.tensor([-40.0, 40.0, 1.25, -1.25]).to(dtype)
    gd, ud = gate.double().numpy(), up.double().numpy()
    gc = np.minimum(gd, limit)
    ref = gc * pp.sigmoid(1.702 * gc) * (np.clip(ud, -limit, limit) + 1.0)
    packed = torch.stack([gate, up], dim=2).reshape(R, 2 * I) if alternating else torch.cat([gate, up], dim=1)
    out = ops().glu_clamped(packed.contiguous().to(DEV), 1.702, limit, alternating=alternating)
    assert relerr(out, ref) < (3e-6 if dtype == torch.float32 else 8e-3)
    assert abs(float(out[0, 0])) < 1e-6  # a gate far below zero: nothing passes


@pytest.mark.parametrize("R,I,K", [(1, 96, 64), (8, 320, 256), (33, 52, 128), (64, 1024, 512)])
def test_the_activation_as_the_products_epilogue(R, I, K):
    """A few bfloat16 rows: the product kernel applies the clamped gated activation
    itself; the same numbers as product, then activation."""
    g = torch.Generator().manual_seed(R + I)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=g) * 0.3).to(torch.bfloat16)  # rows alternate gate, up
    z = x.double().numpy() @ w.double().numpy().T
    gc = np.minimum(z[:, 0::2], 0.9)
    ref = gc * pp.sigmoid(1.702 * gc) * (np.clip(z[:, 1::2], -0.9, 0.9) + 1.0)
    out = ops().linear_glu_clamped(x.to(DEV), w.to(DEV), 1.702, 0.9)
    ops().check_device_errors(DEV)
    assert relerr(out, ref) < 8e-3
    assert np.abs(ref).max() > 0.5 and (np.abs(z[:, 1::2]) > 0.9).mean() > 0.2  # the clamps bite


def test_stream_mix_input_row_gates_and_the_logit_cap():
    g = torch.Generator().manual_seed(2)
    R, H = 5, 24
    x, d, x0 = (torch.randn(R, H, generator=g) for _ in range(3))
    for dt in (torch.float32, torch.bfloat16):
        both = ops().stream_concat(x.to(DEV), d.to(dt).to(DEV), x0.to(DEV), dt).float().cpu()
        want = torch.cat([x + d.to(dt).float(), x0], dim=1).to(dt).float()
        assert torch.equal(both, want)
        assert torch.equal(ops().stream_concat(x.to(DEV), None, x0.to(DEV), dt).float().cpu(),
                           torch.cat([x, x0], dim=1).to(dt).float())
    y, s, z = torch.randn(R, H, generator=g), torch.randn(R, H, generator=g), torch.randn(R, 4, generator=g) * 3
    out = ops().row_gate_add_(y.clone().to(DEV), s.to(DEV), z.to(DEV), 3)
    want = y.double().numpy() + pp.sigmoid(z.double().numpy()[:, 3:4]) * s.double().numpy()
    assert relerr(out, want) < 3e-6
    out = ops().row_gate_add_(y.clone().to(DEV), s.to(DEV), z.to(DEV), 3, extra=x0.to(DEV))
    assert relerr(out, want + x0.double().numpy()) < 3e-6
    lg = torch.randn(3, 50, generator=g) * 40
    out = ops().logit_finish_(lg.clone().to(DEV), 0.5, 30.0)
    assert relerr(out, 30.0 * np.tanh(lg.double().numpy() * 0.5 / 30.0)) < 3e-6
    assert relerr(ops().logit_finish_(lg.clone().to(DEV), 0.5, 0.0), lg.double().numpy() * 0.5) < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,E,top,ff,H,shared", [(1, 5, 2, 24, 64, 40), (9, 3, 3, 40, 72, 0), (70, 8, 1, 16, 100, 24),
                                                 (5, 33, 4, 32, 128, 64), (200, 6, 2, 64, 128, 16), (2, 1, 1, 8, 16, 8)])
def test_experts_with_sigmoid_scores_on_their_inputs_and_a_shared_expert(dtype, R, E, top, ff, H, shared):
    """The part itself (router, route, experts in both forms, shared expert and
    its gate) against the plain feed-forward."""
    from reflex_b200.config.spec import FeedForwardSpec
    from reflex_b200.parts.moe import MixtureOfExperts

    g = torch.Generator().manual_seed(E + top)
    x = torch.randn(R, H, generator=g).to(dtype)
    w = {"router": (torch.randn(E, H, generator=g) / 2).to(dtype)}
    for e in range(E):
        for k, shape in (("gate", (ff, H)), ("up", (ff, H)), ("down", (H, ff))):
            w[f"e{e}.{k}"] = (torch.randn(*shape, generator=g) / 3).to(dtype)
    if shared:
        for k, shape in (("gate", (shared, H)), ("up", (shared, H)), ("down", (H, shared)), ("sg", (1, H))):
            w[f"shared.{k}"] = (torch.randn(*shape, generator=g) / 3).to(dtype)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 1.3}}
    if shared:
        mlp["shared"] = {"ff": shared, "limit": 0.9}
    ref = pp.moe_ff(x.double().numpy(), {k: v.double().numpy() for k, v in w.items()}, "", mlp)
    spec = FeedForwardSpec("moe", H, ff, params=(
        ("experts", E), ("top", top), ("activation", "glu_clamped"), ("alpha", 1.702), ("limit", 1.3),
        ("scores", "sigmoid"), ("weight_input", True), ("shared_ff", shared), ("shared_limit", 0.9)))
    part = MixtureOfExperts(spec, dtype, DEV)
    tensors = {"router": w["router"]}
    for e in range(E):
        tensors.update({f"expert_gate#{e}": w[f"e{e}.gate"], f"expert_up#{e}": w[f"e{e}.up"],
                        f"expert_down#{e}": w[f"e{e}.down"]})
    if shared:
        tensors.update({f"shared_{k}": w[f"shared.{k}"] for k in ("gate", "up", "down", "sg")})
    assert set(tensors) == set(MixtureOfExperts.tensor_specs(spec))
    part.bind(tensors)
    out = part.forward(x.to(DEV))
    assert relerr(out, ref) < (5e-6 if dtype == torch.float32 else 2e-2)
    # the scores: sigmoids of the chosen logits as they are
    logits = f32(x.double().numpy() @ w["router"].double().numpy().T)
    ids, wts = ops().moe_route(logits, None, top, scores="sigmoid")
    z = logits.cpu().double().numpy()
    for r in range(R):
        order = np.argsort(-z[r], kind="stable")[:top]
        assert ids[r].cpu().tolist() == order.tolist()
        assert np.abs(wts[r].cpu().double().numpy() - pp.sigmoid(z[r, order])).max() < 1e-6


# ------------------------------------------------------------ whole models
def make_engine(name, dtype, max_tokens=4096, **kw):
    import reflex_b200
    from reflex_b200.engine import Engine

    model = reflex_b200.load_model(pm.model_folder(name), dtype, DEV)
    return Engine(model, max_tokens=max_tokens, **kw)


_PLAIN = {}


def plain_logits(name, toks):
    key = (name, tuple(toks))
    if key not in _PLAIN:
        cfg, w = pp.read_model(pm.model_folder(name))
        _PLAIN[key] = pp.forward(cfg, w, toks)
    return _PLAIN[key]


def run_cut(engine, toks, cuts):
    """One sequence fed in steps of the given sizes (the last size repeats)."""
    s = engine.open()
    outs, at, i = [], 0, 0
    while at < len(toks):
        n = min(cuts[min(i, len(cuts) - 1)], len(toks) - at)
        outs.append(engine.step([(s, toks[at:at + n], list(range(n)))]).float().cpu().numpy())
        at += n
        i += 1
    engine.close(s)
    return np.concatenate(outs)


def check_rows(got, ref, dtype, what=""):
    scale = np.abs(ref).max()
    err = np.abs(got - ref).max(axis=1) / scale
    if dtype == "float32":
        assert err.max() < 2e-4, (what, int(err.argmax()), float(err.max()))
    else:
        # bfloat16 rounding moves a close router call now and then: nearly all rows are near
        assert (np.median(err) < 4e-2 or len(err) < 8) and (err > 0.12).sum() <= max(1, 0.05 * len(err)), \
            (what, int(err.argmax()), float(err.max()))


LENGTHS = {"A": 150, "B": 200, "C": 140, "D": 280, "E": 140}


def test_layer_by_layer_against_the_plain_model():
    """The residual stream after every layer run of a looped model, 32-bit."""
    from reflex_b200.parts import block

    eng = make_engine("A", "float32")
    toks = pm.tokens(40, pm.ALL["A"]["vocab"], 3)
    cfg, w = pp.read_model(pm.model_folder("A"))
    ref = []
    pp.forward(cfg, w, toks, ref)
    seen = []
    real = block.ParallelBlock.forward

    def spy(self, hidden, pending, ctx, next_norm=None):
        h, d = real(self, hidden, pending, ctx, next_norm)
        seen.append((h + d).cpu().double().numpy())
        return h, d

    block.ParallelBlock.forward = spy
    try:
        s = eng.open()
        eng.step([(s, toks, [0])])
        eng.close(s)
    finally:
        block.ParallelBlock.forward = real
    assert len(seen) == len(ref) == 5
    for i, (a, b) in enumerate(zip(seen, ref)):
        assert np.abs(a - b).max() / np.abs(b).max() < 2e-5, i


@pytest.mark.parametrize("name", sorted(pm.ALL))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_token_by_token_equal_the_plain_model(name, dtype):
    """Each position's logits, with the prompt in one step, token by token from
    the very first token, and in portions of several sizes down to two tokens:
    the filters' look back, the temperature's steps, every page's edge and the
    first tokens are met both inside a prompt and in decoding."""
    eng = make_engine(name, dtype)
    toks = pm.tokens(LENGTHS[name], pm.ALL[name]["vocab"], 11)
    ref = plain_logits(name, toks)
    whole = run_cut(eng, toks, [len(toks)])
    check_rows(whole, ref, dtype, "whole")
    for cuts in ([1], [2], [63, 2, 1, 64, 5], [len(toks) - 40, 1]):
        got = run_cut(eng, toks, cuts)
        check_rows(got, ref, dtype, f"cuts {cuts}")
        if dtype == "float32":
            assert np.abs(got - whole).max() / np.abs(ref).max() < 1e-4


@pytest.mark.parametrize("name", ["A", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_in_reused_slots_equal_each_request_alone(name, dtype):
    """Batches of unequal requests, one after another in a small cache, so that
    slots, pages and state vectors are given back and taken again; shorter
    requests end early."""
    vocab = pm.ALL[name]["vocab"]
    lens = [1, 70, 3, 131, 64, 9, 200, 2]
    reqs = [pm.tokens(n, vocab, 20 + i) for i, n in enumerate(lens)]
    eng = make_engine(name, dtype, max_tokens=640, max_slots=3, use_graphs=(name == "A"))
    for b0 in range(0, len(reqs), 3):
        idx = list(range(b0, min(len(reqs), b0 + 3)))
        seqs = {i: eng.open() for i in idx}
        fed = {i: 0 for i in idx}
        got = {i: [] for i in idx}
        first = True
        while seqs:
            order = list(seqs)
            entries = []
            for i in order:
                n = max(1, len(reqs[i]) - 20) if first else 1
                part = reqs[i][fed[i]:fed[i] + n]
                entries.append((seqs[i], part, list(range(len(part)))))
            out = eng.step(entries).float().cpu().numpy()
            r = 0
            for i, e in zip(order, entries):
                got[i].append(out[r:r + len(e[1])])
                r += len(e[1])
                fed[i] += len(e[1])
                if fed[i] == len(reqs[i]):
                    eng.close(seqs.pop(i))
            first = False
        for i in idx:
            check_rows(np.concatenate(got[i]), plain_logits(name, reqs[i]), dtype, f"request {i}")
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_pages(dtype):
    """A short prompt and 700 decoded tokens: the recurrence's state and the
    filters' last inputs are carried for hundreds of steps, the temperature
    steps a hundred times, and the flat heads still see the first tokens from
    eleven pages away."""
    eng = make_engine("A", dtype, max_tokens=1024)
    toks = pm.tokens(710, pm.ALL["A"]["vocab"], 5)
    ref = plain_logits("A", toks)
    got = run_cut(eng, toks, [10, 1])
    check_rows(got, ref, dtype, "long decode")


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_greedy_generation_through_the_entry_point(dtype):
    """`Model.generate` (the scheduler, the sampler, decode graphs in bfloat16)
    against greedy continuation by the plain model."""
    import reflex_b200

    name = "D"
    model = reflex_b200.Model.load(pm.model_folder(name), weights=dtype, max_tokens=2048, max_batch=3)
    vocab = pm.ALL[name]["vocab"]
    prompts = [pm.tokens(n, vocab, 40 + n) for n in (5, 70, 1, 130)]
    n_new = 12
    got = model.generate(prompts, n_new)
    cfg, w = pp.read_model(pm.model_folder(name))
    for p, out in zip(prompts, got):
        assert len(out) == n_new
        seq = list(p)
        for t, tok in enumerate(out):
            lg = pp.forward(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if dtype == "bf16" and top2[1] - top2[0] < 0.15 * np.abs(lg).max():
                break  # a near tie: bfloat16 may pick the other one, and the continuations part
            assert tok == int(np.nonzero(lg == lg.max())[0][-1]), (len(p), t)
            seq.append(tok)


def test_candidate_scores_carry_the_scale_and_the_cap():
    """`Engine.step_scores` (one given id per wanted place) gives the capped
    logit of that id, as the full-vocabulary step does."""
    eng = make_engine("C", "float32")
    toks = pm.tokens(30, pm.ALL["C"]["vocab"], 2)
    ref = plain_logits("C", toks)
    s = eng.open()
    ids = [5, 17, 60]
    out = eng.step_scores([(s, toks, [0, 12, 29], ids)]).cpu().double().numpy()
    eng.close(s)
    want = np.array([ref[0, 5], ref[12, 17], ref[29, 60]])
    assert np.abs(out - want).max() / np.abs(ref).max() < 2e-4
