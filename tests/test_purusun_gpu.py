"""Purusun on the GPU: every mechanism alone against the plain implementation
(`plain_purusun`), then whole models through the engine under every way of
cutting the work, and generation through the entry point."""

import math

import numpy as np
import pytest
import torch

import plain_purusun as pp
import purusun_models as pm
from test_kegasun_gpu import FakeBatch, i32, ops, relerr
from test_kernels_gpu import _paged

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def f32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


# ------------------------------------------------------------- mechanisms
@pytest.mark.parametrize("S,W,R", [(1, 64, 3), (2, 100, 5), (3, 328, 70), (4, 4096, 2), (8, 72, 9), (3, 1028, 5),
                                   (2, 2048, 33), (1, 1024, 32), (8, 1536, 1)])
@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_streams_write_read_norm_and_sum(S, W, R, y_dtype, out_dtype):
    """One launch: the write of the sublayer before (mix [from, to], a per-channel
    scale), the read and its norm with a 1 + w weight; then the last write and
    the sum of the streams."""
    g = torch.Generator().manual_seed(S * 1000 + W)
    x0 = torch.randn(R, W, generator=g)
    xs = ops().hyper_expand(x0.to(DEV), S)
    assert torch.equal(xs.cpu(), x0.repeat(1, S).reshape(R, S * W))
    xs = (xs + torch.randn(R, S * W, generator=g).to(DEV)).contiguous()  # streams that differ
    ref = xs.cpu().double().numpy().reshape(R, S, W).transpose(1, 0, 2)
    y = torch.randn(R, W, generator=g).to(y_dtype)
    ls, mix = torch.rand(W, generator=g) + 0.5, torch.randn(S, S, generator=g)
    wout, win, nw = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(W, generator=g) * 0.1
    tol = 3e-6 if out_dtype == torch.float32 else 8e-3
    # a read alone
    out = ops().hyper_step(xs, None, win.to(DEV), nw.to(DEV), 1e-5, 1.0, out_dtype, S)
    assert relerr(out, pp.norm_one_plus(pp.hyper_read(ref, win.double().numpy()), nw.double().numpy(), 1e-5)) < tol
    assert np.array_equal(xs.cpu().double().numpy().reshape(R, S, W).transpose(1, 0, 2), ref)  # untouched
    # write, then read
    write = ops().StreamWrite(y.to(DEV), ls.to(DEV), mix.to(DEV).contiguous(), wout.to(DEV))
    total = ops().hyper_collapse(xs, write, S)  # leaves the streams alone
    out = ops().hyper_step(xs, write, win.to(DEV), nw.to(DEV), 1e-5, 1.0, out_dtype, S)
    new = pp.hyper_write(ref, y.double().numpy() * ls.double().numpy(), mix.double().numpy(), wout.double().numpy())
    assert relerr(xs.reshape(R, S, W).transpose(0, 1), new) < 3e-6
    assert relerr(out, pp.norm_one_plus(pp.hyper_read(new, win.double().numpy()), nw.double().numpy(), 1e-5)) < tol
    assert relerr(total, new.sum(axis=0)) < 3e-6
    assert relerr(ops().hyper_collapse(xs, None, S), new.sum(axis=0)) < 3e-6
    # only some rows, in an order of their own, with the write still to come
    pick = [R - 1, 0, R // 2]
    xs3 = torch.tensor(ref.transpose(1, 0, 2).reshape(R, S * W), dtype=torch.float32, device=DEV)
    some = ops().hyper_collapse(xs3, write, S, rows=i32(pick))
    assert tuple(some.shape) == (3, W) and relerr(some, new.sum(axis=0)[pick]) < 3e-6
    # no scale: y as it is
    xs2 = torch.tensor(ref.transpose(1, 0, 2).reshape(R, S * W), dtype=torch.float32, device=DEV)
    write = ops().StreamWrite(y.to(DEV), None, mix.to(DEV).contiguous(), wout.to(DEV))
    ops().hyper_step(xs2, write, win.to(DEV), nw.to(DEV), 1e-5, 0.0, out_dtype, S)
    new = pp.hyper_write(ref, y.double().numpy(), mix.double().numpy(), wout.double().numpy())
    assert relerr(xs2.reshape(R, S, W).transpose(0, 1), new) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,rot,extra", [
    (4, 2, 16, (100.0, 8, (8.0, 1.0, 4.0, 64)), 64), (3, 3, 40, (1000.0, 20, (2.0, 0.5, 2.0, 32)), 120),
    (8, 2, 128, (500000.0, 32, (4.0, 1.0, 4.0, 128)), 0), (2, 1, 64, (10000.0, 64, None), 128),
    (1, 1, 12, None, 5)])
def test_keys_as_values_partial_scaled_rotation_and_the_cache_write(dtype, nq, nkv, d, rot, extra):
    """Rows of a stacked product [q | k | further columns]: q and k normed per head
    with one plain weight and rotated on their first dimensions with the scaled
    frequencies; the values written to the cache are the keys as projected.
    Positions far out (large angles), at a page's edge and at zero."""
    from reflex_b200.config.spec import PositionSpec
    from reflex_b200.parts.registry import POSITIONS

    g = torch.Generator().manual_seed(nq + d)
    pos = [0, 1, 63, 64, 65, 1000, 4099]
    R = len(pos)
    ld = (nq + nkv) * d
    proj = torch.randn(R, ld + extra, generator=g) * 2
    qw, kw = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    rotation, freqs = None, np.zeros(0)
    if rot is not None:
        base, dims, sc = rot
        spec = PositionSpec("rope_scaled" if sc else "rope_neox", d, dims, base,
                            tuple(zip(("factor", "low", "high", "original"), sc)) if sc else ())
        rotation = POSITIONS.get(spec.kind)(spec, dtype, DEV).rotation()
        freqs = pp.rotary_frequencies(dims, base, dict(zip(("factor", "low", "high", "original"), sc)) if sc else None)
        assert relerr(1.0 / rotation.denominators, freqs) < 1e-6
    n_pages = 4099 // 64 + 1
    table = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, n_pages).contiguous()
    kp = torch.zeros(n_pages, nkv, 64, d, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    src = proj.to(dtype)
    q = ops().qkv_post(src.to(DEV), qw.to(DEV), kw.to(DEV), 1e-5, 0.0, rotation, i32(pos), i32([0] * R), kp, vp,
                       table.to(DEV), 64, nq, nkv, d, True, dtype, values_are_keys=True, ld=ld)
    x = src.double().numpy()
    qr = pp.rotate(pp.rms_unit(x[:, :nq * d].reshape(R, nq, d), 1e-5) * qw.double().numpy(), np.array(pos), freqs)
    kraw = x[:, nq * d:ld].reshape(R, nkv, d)
    kr = pp.rotate(pp.rms_unit(kraw, 1e-5) * kw.double().numpy(), np.array(pos), freqs)
    # 32-bit angles: at position 4,099 an angle of thousands of radians is known to a few 1e-4 of one
    tol = 1e-4 if dtype == torch.float32 else 8e-3
    assert relerr(q.reshape(R, nq, d), qr) < tol
    for r, p in enumerate(pos):
        page = int(table[0, p // 64])
        assert relerr(kp[page, :, p % 64], kr[r]) < tol, p
        assert relerr(vp[page, :, p % 64], kraw[r]) < (1e-7 if dtype == torch.float32 else 1e-7), p  # a copy


def _kept_ref(q, ks, vs, seqs, scale, window, keep, dtype):
    outs, r = [], 0
    for (start, n), k, v in zip(seqs, ks, vs):
        kk, vv = k.to(dtype).double().numpy(), v.to(dtype).double().numpy()
        for t in range(n):
            i = start + t
            js = [j for j in range(i + 1) if pp.visible(i, j, window, keep)]
            o = np.zeros((q.shape[1], vv.shape[2]))
            for h in range(q.shape[1]):
                kvh = h // (q.shape[1] // kk.shape[1])
                s = (kk[js, kvh] @ q[r + t, h].to(dtype).double().numpy()) * scale
                e = np.exp(s - s.max())
                o[h] = (e[:, None] * vv[js, kvh]).sum(0) / e.sum()
            outs.append(o)
        r += n
    return np.stack(outs)


KEPT_CASES = [  # nq, nkv, d, [(start, n_new)], window, keep_first
    (4, 2, 16, [(0, 70), (130, 3), (0, 1)], 20, 3),
    (2, 1, 64, [(0, 200), (63, 2), (133, 3)], 70, 65),     # kept tokens reach into a second page
    (6, 1, 64, [(0, 400), (328, 4)], 200, 130),            # into a third; position 329 is the first to lose one
    (8, 2, 128, [(0, 150), (200, 40)], 33, 1),
    (3, 3, 40, [(0, 140)], 64, 0),                         # a window of a page, nothing kept
    (12, 3, 128, [(0, 300)], 150, 5),
    (4, 4, 32, [(0, 100), (30, 50)], 5, 64),               # more kept than the window is long
]


@pytest.mark.parametrize("kernel", ["plain_f32", "plain_bf16", "prefill_bf16", "prefill_tc_bf16", "decode_bf16",
                                    "dispatch_bf16"])
@pytest.mark.parametrize("nq,nkv,d,seqs,window,keep", KEPT_CASES)
def test_a_window_that_keeps_the_first_tokens_in_every_attention_kernel(kernel, nq, nkv, d, seqs, window, keep):
    """i sees j iff j <= i and (i - j < window or j < keep_first).  The last kept
    key and the first one that is not kept are made to stand out (large
    multiples of the mean query), and so are the keys just inside and just
    outside the window of the last row: one token off anywhere moves the
    result by whole units."""
    if not kernel.startswith("plain") and d % 16:
        pytest.skip("multiples of 16")
    if kernel == "prefill_tc_bf16" and d not in (64, 128):
        pytest.skip("head sizes 64 and 128")
    g = torch.Generator().manual_seed(nq + d + keep)
    dtype = torch.float32 if kernel == "plain_f32" else torch.bfloat16
    if kernel == "decode_bf16":
        seqs = [(a + b - 1, 1) for a, b in seqs]
    slots, table, kp, vp, ks, vs = _paged([a + b for a, b in seqs], nkv, d, dtype, g)
    R = sum(b for _, b in seqs)
    q = torch.randn(R, nq, d, generator=g) + 1.0
    scale = d ** -0.5
    loud = torch.ones(d) * (9.0 / (scale * d))  # along the queries' common direction: about 9 units of score
    kd_host = kp.clone()
    for i, (a, b) in enumerate(seqs):
        last = a + b - 1
        for j in (keep - 1, keep, last - window, last - window + 1):
            if 0 <= j <= last:
                ks[i][j] = loud
                kd_host[int(table[slots[i], j // 64]), :, j % 64] = loud.to(dtype)
    ref = _kept_ref(q, ks, vs, seqs, scale, window, keep, dtype)
    if keep:
        assert np.abs(ref - _kept_ref(q, ks, vs, seqs, scale, window, keep - 1, dtype)).max() > 0.2
    assert np.abs(ref - _kept_ref(q, ks, vs, seqs, scale, window + 1, keep, dtype)).max() > 0.2
    qd = q.reshape(R, nq * d).to(dtype).to(DEV)
    kd, vd, td = kd_host.to(DEV), vp.to(DEV), table.to(DEV)
    row_pos = i32([a + j for a, b in seqs for j in range(b)])
    row_slot = i32([slots[i] for i, (a, b) in enumerate(seqs) for _ in range(b)])
    outs = []
    if kernel.startswith("plain"):
        outs.append(ops().attention_plain(qd, kd, vd, td, 64, row_pos, row_slot, nq, nkv, d, window, scale,
                                          keep_first=keep))
    elif kernel == "decode_bf16":
        for splits in (1, 2, 3, 4):  # alone, merged inside a cluster, merged by the combine kernel
            outs.append(ops().attention_decode(qd, kd, vd, td, 64, row_pos, row_slot, nq, nkv, d, window, scale,
                                               n_splits=splits, keep_first=keep))
    else:
        row0 = [0]
        for _, b in seqs:
            row0.append(row0[-1] + b)
        if kernel == "dispatch_bf16":  # what a model's step calls: picks the kernel itself
            b = FakeBatch([[0] * n for _, n in seqs], slots, [a for a, _ in seqs])
            b.is_decode, b.max_new = False, max(n for _, n in seqs)
            b.max_context = max(a + n for a, n in seqs)
            outs.append(ops().attention(qd, kd, vd, td, 64, b, nq, nkv, d, window, scale, keep_first=keep))
        else:
            fn = ops().attention_prefill_tc if kernel == "prefill_tc_bf16" else ops().attention_prefill
            outs.append(fn(qd, kd, vd, td, 64, i32(slots), i32([a for a, _ in seqs]), i32([b for _, b in seqs]),
                           i32(row0), max(b for _, b in seqs), nq, nkv, d, window, scale, keep_first=keep))
    ops().check_device_errors(DEV)
    for out in outs:
        assert not bool(torch.isnan(out.float()).any())
        assert relerr(out.reshape(R, nq, d), ref) < (3e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("a_dtype,z_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                             (torch.bfloat16, torch.bfloat16)])
def test_sigmoid_gate_from_columns_of_a_wider_row_and_squared_relu(a_dtype, z_dtype):
    g = torch.Generator().manual_seed(5)
    for R, H, col, ld in ((1, 640, 896, 1600), (70, 52, 9, 70), (9, 4096, 0, 4096)):
        a = torch.randn(R, H, generator=g).to(a_dtype)
        z = (torch.randn(R, ld, generator=g) * 4).to(z_dtype)
        ref = a.double().numpy() * pp.sigmoid(z[:, col:col + H].double().numpy())
        out = ops().sigmoid_gate_mul_(a.to(DEV), z.to(DEV), col)
        assert relerr(out, ref) < (3e-6 if a_dtype == torch.float32 else 8e-3)
        x = (torch.randn(R, H, generator=g) * 3).to(a_dtype)
        assert relerr(ops().relu2_(x.to(DEV).clone()), np.maximum(x.double().numpy(), 0.0) ** 2) < \
            (1e-6 if a_dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("R,N,K", [(1, 96, 64), (8, 1000, 328), (33, 256, 2048), (64, 152, 72), (65, 64, 64), (3, 77, 64), (5, 250, 200)])
def test_squared_relu_as_the_products_epilogue(R, N, K):
    """A few bfloat16 rows: the activation rides in the product kernel; beyond, apart."""
    g = torch.Generator().manual_seed(R + N)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    prod = x.double().numpy() @ w.double().numpy().T
    ref = np.maximum(prod, 0.0) ** 2
    out = ops().linear_relu2(x.to(DEV), w.to(DEV))
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (R, N)
    assert relerr(out, ref) < 8e-3
    # the signs: where the product is clearly negative the result is exactly zero
    assert bool((out.cpu().double().numpy()[prod < -1e-2] == 0.0).all())


# rows per sequence and step; the first step is long enough for the scan to cut its sequences
# into segments (also the one of nine rows), the last but one for one sequence in three
CUTS = ({0: 197, 1: 9, 2: 81}, {0: 1, 2: 2}, {2: 1}, {0: 2, 2: 14}, {2: 1, 0: 1}, {2: 115}, {0: 1, 2: 1}, {0: 30})


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,N,taps", [(48, 8, 3), (24, 1, 1), (50, 5, 5), (256, 64, 4), (16, 130, 2), (36, 16, 4),
                                      (8, 300, 2), (21, 32, 3)])
@pytest.mark.parametrize("gap", [1, 4])
def test_filter_silu_and_scan_carried_through_their_state(C, N, taps, out_dtype, gap):
    """Three sequences of unequal lengths in steps of unequal sizes, down to one
    and two rows, in slots that are not in order: the filter's last inputs and
    the scan's state go on from what the steps before left; a slot taken again
    starts from zeros.  Step sizes from nearly zero to several units.  B and C
    lie `gap` floats into their rows and apart (4: every address a multiple of
    16 bytes where the sizes allow it; 1: none)."""
    g = torch.Generator().manual_seed(C + N)
    b_off, c_off, ld_bc = gap, N + 2 * gap, 2 * N + 3 * gap
    lens, slots = {0: 232, 1: 9, 2: 215}, {0: 3, 1: 0, 2: 6}
    ld_z, z_off = 2 * C + 4, C + 4
    xz = {s: torch.randn(n, ld_z, generator=g) for s, n in lens.items()}
    dtpre = {s: torch.randn(n, C, generator=g) * 3 for s, n in lens.items()}
    bc = {s: torch.randn(n, ld_bc, generator=g) for s, n in lens.items()}
    w, cb = torch.randn(C, taps, generator=g) * 0.6, torch.randn(C, generator=g) * 0.3
    dtb, A = torch.randn(C, generator=g), -torch.exp(torch.randn(C, N, generator=g) * 0.7)
    D = torch.randn(C, generator=g)
    n_state = (taps - 1) * C + C * N
    state = torch.zeros(8, n_state + 8, device=DEV)
    state[:, n_state:] = 5.0  # floats beside this mixer's
    fed = {s: 0 for s in lens}
    got = {s: [] for s in lens}
    for cuts in CUTS:
        ids = list(cuts)
        b = FakeBatch([[0] * cuts[s] for s in ids], [slots[s] for s in ids], [fed[s] for s in ids])
        cat = lambda d: torch.cat([d[s][fed[s]:fed[s] + cuts[s]] for s in ids]).to(DEV).contiguous()  # noqa: E731
        rows = cat(xz)
        single = all(n == 1 for n in cuts.values())  # a row a sequence: the filter's launch moves its state on
        u = ops().short_conv(rows, 0, C, None, w.t().contiguous().to(DEV), cb.to(DEV), state if taps > 1 else None, b,
                             activation="silu", update_state=single and taps > 1)
        if not single:
            ops().conv_state_update(rows, 0, C, None, taps, state, b)
        y = ops().mamba_scan(u, cat(dtpre), dtb.to(DEV), cat(bc), b_off, c_off, rows, z_off, A.to(DEV).contiguous(),
                             D.to(DEV), state, (taps - 1) * C, b, out_dtype)
        for j, s in enumerate(ids):
            got[s].append(y[b.row0[j]:b.row0[j + 1]].float().cpu())
            fed[s] += cuts[s]

    def ref(s):
        x = pp.silu(pp.causal_conv(xz[s][:, :C].double().numpy(), w.double().numpy(), cb.double().numpy()))
        dt = pp.softplus(dtpre[s].double().numpy() + dtb.double().numpy())
        B, Cm = bc[s][:, b_off:b_off + N].double().numpy(), bc[s][:, c_off:c_off + N].double().numpy()
        y = pp.scan_core(x, dt, A.double().numpy(), B, Cm, D.double().numpy())
        return y * pp.silu(xz[s][:, z_off:z_off + C].double().numpy())

    tol = 2e-5 if out_dtype == torch.float32 else 8e-3
    for s in lens:
        assert fed[s] == lens[s]
        assert relerr(torch.cat(got[s]), ref(s)) < tol, s
    assert bool((state[:, n_state:] == 5.0).all())
    # a slot taken again: zeros, as the cache leaves it
    state[0].zero_()
    b = FakeBatch([[0] * 9], [0], [0])
    rows = xz[1].to(DEV)
    u = ops().short_conv(rows, 0, C, None, w.t().contiguous().to(DEV), cb.to(DEV), state if taps > 1 else None, b,
                         activation="silu")
    y = ops().mamba_scan(u, dtpre[1].to(DEV), dtb.to(DEV), bc[1].to(DEV), b_off, c_off, rows, z_off,
                         A.to(DEV).contiguous(), D.to(DEV), state, (taps - 1) * C, b, out_dtype)
    assert relerr(y, ref(1)) < tol


@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,N,rank,rows", [(48, 8, 4, 1), (24, 1, 1, 1), (50, 5, 3, 1), (256, 64, 8, 1), (16, 130, 2, 1),
                                           (40, 16, 128, 2)])
def test_step_sizes_from_their_low_rank_vector_inside_the_scan(C, N, rank, rows, w_dtype):
    """A row or two a sequence: the rows hold [vector | B | C]; the kernel makes
    W_dt . vector itself (the vector rounded to bfloat16 where the weights are)."""
    g = torch.Generator().manual_seed(C * 7 + N)
    n_seq, ld = 3, rank + 2 * N
    R = n_seq * rows
    u, xz = torch.randn(R, C, generator=g), torch.randn(R, 2 * C, generator=g)
    proj = torch.randn(R, ld, generator=g)
    w_dt = (torch.randn(C, rank, generator=g) * 2 / math.sqrt(rank)).to(w_dtype)
    dtb, A = torch.randn(C, generator=g), -torch.exp(torch.randn(C, N, generator=g) * 0.7)
    D = torch.randn(C, generator=g)
    state0 = torch.randn(4, C * N + 3, generator=g)
    b = FakeBatch([[0] * rows] * n_seq, [2, 0, 3], [5, 6, 7])
    low = proj[:, :rank].to(w_dtype).double().numpy()
    dtpre = low @ w_dt.double().numpy().T
    st1, st2 = state0.clone().to(DEV), state0.clone().to(DEV)
    got = ops().mamba_scan(u.to(DEV), None, dtb.to(DEV), proj.to(DEV), rank, rank + N, xz.to(DEV), C,
                           A.to(DEV).contiguous(), D.to(DEV), st1, 0, b, torch.float32, dt_weight=w_dt.to(DEV),
                           dt_low_off=0)
    want = ops().mamba_scan(u.to(DEV), torch.tensor(dtpre, dtype=torch.float32, device=DEV), dtb.to(DEV), proj.to(DEV),
                            rank, rank + N, xz.to(DEV), C, A.to(DEV).contiguous(), D.to(DEV), st2, 0, b, torch.float32)
    assert relerr(got, want.double().cpu().numpy()) < 2e-5
    assert relerr(st1, st2.double().cpu().numpy()) < 2e-5
    # and against the recurrence written out, from the states the slots held
    for j, slot in enumerate([2, 0, 3]):
        S = state0[slot, :C * N].double().numpy().reshape(C, N).copy()
        for t in range(rows):
            r = j * rows + t
            dt = pp.softplus(dtpre[r] + dtb.double().numpy())
            S = np.exp(dt[:, None] * A.double().numpy()) * S + (dt * u[r].double().numpy())[:, None] * \
                proj[r, rank:rank + N].double().numpy()[None, :]
            y = S @ proj[r, rank + N:].double().numpy() + D.double().numpy() * u[r].double().numpy()
            assert relerr(got[r], y * pp.silu(xz[r, C:].double().numpy())) < 2e-5, (slot, t)


def test_a_slow_decay_keeps_a_far_input_and_a_fast_one_forgets_it():
    """One large input at the first token, 600 tokens of nothing after it: the
    channel whose decay is nearly one still holds it, the fast one has lost it;
    token by token through the state."""
    C, N, T = 4, 2, 600
    x = torch.zeros(T, C)
    x[0] = 5.0
    dtpre = torch.full((T, C), 0.0)
    bc = torch.ones(T, 2 * N)
    A = torch.tensor([[-1e-4, -1e-3], [-1e-2, -0.05], [-0.5, -1.0], [-3.0, -8.0]])
    z = torch.full((T, C), 30.0)  # silu(30) = 30
    state = torch.zeros(2, C * N, device=DEV)
    outs = []
    for t0, n in ((0, 1), (1, 299), (300, 1), (301, 299)):
        b = FakeBatch([[0] * n], [1], [t0])
        outs.append(ops().mamba_scan(x[t0:t0 + n].to(DEV).contiguous(), dtpre[t0:t0 + n].to(DEV).contiguous(), None,
                                     bc[t0:t0 + n].to(DEV).contiguous(), 0, N, z[t0:t0 + n].to(DEV).contiguous(), 0,
                                     A.to(DEV), None, state, 0, b, torch.float32).cpu())
    y = torch.cat(outs).double().numpy()
    dt = pp.softplus(np.zeros((T, C)))
    ref = pp.scan_core(x.double().numpy(), dt, A.double().numpy(), np.ones((T, N)), np.ones((T, N)), np.zeros(C)) * 30.0
    # 600 decays in 32-bit, each rounded: a few 1e-5 in all
    assert np.abs(y - ref).max() / np.abs(ref).max() < 5e-5
    assert ref[-1, 0] > 0.75 * ref[0, 0] and abs(ref[-1, 3]) < 1e-30 and abs(y[-1, 3]) < 1e-30
    assert abs(y[-1, 0] - ref[-1, 0]) / ref[-1, 0] < 5e-5


# ----------------------------------------------------------------- whole models
def sharpness(dtype):
    """The full factors in 32-bit; their square roots in bfloat16 (`purusun_models.model_folder`)."""
    return True if dtype in ("float32", "f32") else "mild"


def make_engine(name, dtype, max_tokens=4096, **kw):
    import reflex_b200
    from reflex_b200.engine import Engine

    model = reflex_b200.load_model(pm.model_folder(name, sharp=sharpness(dtype)), dtype, DEV)
    return Engine(model, max_tokens=max_tokens, **kw)


_PLAIN = {}


def plain_logits(name, toks, dtype="float32"):
    key = (name, tuple(toks), sharpness(dtype))
    if key not in _PLAIN:
        cfg, w = pp.read_model(pm.model_folder(name, sharp=sharpness(dtype)))
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
        assert (np.median(err) < 4e-2 or len(err) < 8) and (err > 0.12).sum() <= max(1, 0.05 * len(err)), \
            (what, int(err.argmax()), float(err.max()), float(np.median(err)))


LENGTHS = {"A": 170, "B": 140, "C": 150, "D": 150, "E": 300}


@pytest.mark.parametrize("name", ["A", "C"])
def test_layer_by_layer_against_the_plain_model(name):
    """The sum of the residual streams after every layer run of a looped model, 32-bit."""
    eng = make_engine(name, "float32")
    model = eng.model
    toks = pm.tokens(40, pm.ALL[name]["vocab"], 3)
    cfg, w = pp.read_model(pm.model_folder(name))
    _logits, ref = pp.forward(cfg, w, toks, want_layers=True)
    seen = []

    def after(i, run, layer, h, pending):
        seen.append(ops().hyper_collapse(h, layer._pending_write(h, pending), model.spec.residual_streams)
                    .cpu().double().numpy())

    model.after_run = after
    s = eng.open()
    eng.step([(s, toks, [0])])
    eng.close(s)
    model.after_run = None
    assert len(seen) == len(ref) == 5
    for i, (a, b) in enumerate(zip(seen, ref)):
        assert np.abs(a - b).max() / np.abs(b).max() < 5e-5, (i, np.abs(a - b).max() / np.abs(b).max())


@pytest.mark.parametrize("name", sorted(pm.ALL))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_token_by_token_equal_the_plain_model(name, dtype):
    """Each position's logits, with the prompt in one step, token by token from
    the very first token, and in portions of several sizes down to two tokens:
    the windows' edges, the kept first tokens, the filters' look back, every
    page's edge and the first tokens are met both inside a prompt and in
    decoding."""
    eng = make_engine(name, dtype)
    toks = pm.tokens(LENGTHS[name], pm.ALL[name]["vocab"], 11)
    ref = plain_logits(name, toks, dtype)
    whole = run_cut(eng, toks, [len(toks)])
    check_rows(whole, ref, dtype, "whole")
    for cuts in ([1], [2], [63, 2, 1, 64, 5], [len(toks) - 40, 1]):
        got = run_cut(eng, toks, cuts)
        check_rows(got, ref, dtype, f"cuts {cuts}")
        if dtype == "float32":
            assert np.abs(got - whole).max() / np.abs(ref).max() < 1e-4
    eng.check_errors()


@pytest.mark.parametrize("name", ["A", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_in_reused_slots_equal_each_request_alone(name, dtype):
    """Batches of unequal requests, one after another in a small cache, so that
    slots, pages and state vectors are given back and taken again; shorter
    requests end early."""
    vocab = pm.ALL[name]["vocab"]
    lens = [1, 70, 3, 131, 64, 9, 200, 2]
    reqs = [pm.tokens(n, vocab, 20 + i) for i, n in enumerate(lens)]
    eng = make_engine(name, dtype, max_tokens=640, max_slots=3, use_graphs=(name != "D"))
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
            check_rows(np.concatenate(got[i]), plain_logits(name, reqs[i], dtype), dtype, f"request {i}")
    assert eng.cache.tokens_held() == 0
    eng.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_pages(dtype):
    """A short prompt and 700 decoded tokens: the scan's state and the filter's
    last inputs are carried for hundreds of steps, both windows pass over
    decoded tokens many times, their pages are given back while the kept first
    pages stay, and the kept tokens are still seen from eleven pages away."""
    eng = make_engine("A", dtype, max_tokens=1024)
    toks = pm.tokens(710, pm.ALL["A"]["vocab"], 5)
    ref = plain_logits("A", toks, dtype)
    got = run_cut(eng, toks, [10, 1])
    check_rows(got, ref, dtype, "long decode")
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_greedy_generation_through_the_entry_point(dtype):
    """`Model.generate` (the scheduler, the sampler, decode graphs in bfloat16)
    against greedy continuation by the plain model."""
    import reflex_b200

    name = "D"
    folder = pm.model_folder(name, sharp=sharpness(dtype))
    model = reflex_b200.Model.load(folder, weights=dtype, max_tokens=2048, max_batch=3)
    vocab = pm.ALL[name]["vocab"]
    prompts = [pm.tokens(n, vocab, 40 + n) for n in (5, 70, 1, 130)]
    n_new = 12
    got = model.generate(prompts, n_new)
    cfg, w = pp.read_model(folder)
    for p, out in zip(prompts, got):
        assert len(out) == n_new
        seq = list(p)
        for t, tok in enumerate(out):
            lg = pp.forward(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if dtype == "bf16" and top2[1] - top2[0] < 0.15 * np.abs(lg).max():
                break  # a near tie: bfloat16 may pick the other one, and the continuations part
            assert tok == pp.argmax_last(lg), (len(p), t)
            seq.append(tok)


def test_decode_steps_are_captured_into_graphs():
    eng = make_engine("E", "bfloat16")
    assert eng.model.capturable and eng.use_graphs
