"""Zelinex on the GPU: every mechanism alone against the plain implementation
(`plain_zelinex`), then whole models through the engine under every way of
cutting the work, and generation through the entry point."""

import math

import numpy as np
import pytest
import torch

import plain_zelinex as pz
import zelinex_models as zm
from test_kegasun_gpu import FakeBatch, i32, ops, relerr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def f32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


def tol(dtype, exact=3e-6, low=8e-3):
    return exact if dtype == torch.float32 else low


# ------------------------------------------------------------- mechanisms
@pytest.mark.parametrize("R,H", [(1, 64), (3, 100), (5, 4096), (70, 72), (2, 20000)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_after_a_sublayer_and_before_the_next_in_one_pass(R, H, out_dtype):
    g = torch.Generator().manual_seed(R + H)
    x, y = torch.randn(R, H, generator=g) * 2, torch.randn(R, H, generator=g) * 5
    wp, wn = torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g) + 0.5
    new = x.double().numpy() + 0.65 * pz.rms_norm(y.double().numpy(), wp.double().numpy(), 1e-5)
    xd = x.to(DEV)
    out = ops().sandwich_norm(y.to(DEV), xd, wp.to(DEV), 0.65, 1e-5, wn.to(DEV), 1e-6, out_dtype)
    assert relerr(xd, new) < 3e-6
    assert relerr(out, pz.rms_norm(new, wn.double().numpy(), 1e-6)) < tol(out_dtype)
    xd = x.to(DEV)
    assert ops().sandwich_norm(y.to(DEV), xd, wp.to(DEV), 0.65, 1e-5, None, 0.0, out_dtype) is None
    assert relerr(xd, new) < 3e-6


@pytest.mark.parametrize("R,C,groups", [(1, 64, 1), (3, 96, 2), (5, 100, 5), (70, 256, 2), (2, 4096, 32), (4, 120, 3)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_in_equal_parts_with_and_without_a_gate(R, C, groups, out_dtype):
    g = torch.Generator().manual_seed(R + C)
    x, w = torch.randn(R, C, generator=g) * 3, torch.rand(C, generator=g) + 0.5
    z = torch.randn(R, C + 24, generator=g) * 3
    ref = pz.rms_unit(x.double().numpy().reshape(R, groups, C // groups), 1e-5).reshape(R, C) * w.double().numpy()
    out = ops().group_norm_gate(x.to(DEV), w.to(DEV), 1e-5, groups, out_dtype)
    assert relerr(out, ref) < tol(out_dtype)
    out = ops().group_norm_gate(x.to(DEV), w.to(DEV), 1e-5, groups, out_dtype, gate=z.to(DEV), gate_col=16)
    assert relerr(out, ref * pz.sigmoid(z.double().numpy()[:, 16:16 + C])) < tol(out_dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_xielu_pass_start_tanh_columns_and_scaled_sum(dtype):
    g = torch.Generator().manual_seed(5)
    z = (torch.randn(7, 333, generator=g) * 4).to(dtype)
    ap, an = float(pz.softplus(0.3)), 0.5 + float(pz.softplus(-0.7))
    out = ops().xielu_(z.clone().to(DEV), ap, an)
    assert relerr(out, pz.xielu(z.double().numpy(), 0.3, -0.7)) < tol(dtype, 2e-6)
    x, x0, v = torch.randn(5, 72, generator=g), torch.randn(5, 72, generator=g), torch.randn(72, generator=g)
    assert relerr(ops().loop_input_(x.clone().to(DEV), x0.to(DEV), v.to(DEV)), (x + x0 + v).double().numpy()) < 1e-6
    assert relerr(ops().loop_input_(x.clone().to(DEV), None, v.to(DEV)), (x + v).double().numpy()) < 1e-6
    rows = torch.randn(6, 50, generator=g) * 2
    assert relerr(ops().tanh_cols(rows.to(DEV), 13, 7, dtype), np.tanh(rows.double().numpy()[:, 13:20])) < tol(dtype, 2e-6)
    a, b = torch.randn(9, 41, generator=g), torch.randn(9, 41, generator=g)
    assert relerr(ops().scaled_sum_(a.clone().to(DEV), b.to(DEV), 0.55, -1.5), (0.55 * a - 1.5 * b).double().numpy()) < 1e-6


@pytest.mark.parametrize("R,N,K", [(1, 96, 64), (8, 1000, 328), (33, 256, 2048), (64, 152, 72), (65, 64, 64), (3, 77, 64),
                                   (5, 250, 200)])
def test_xielu_as_the_products_epilogue(R, N, K):
    """A few bfloat16 rows: the activation rides in the product kernel (on the 32-bit
    sums); more rows, or a width that is no multiple of 8: product, then the kernel."""
    g = torch.Generator().manual_seed(R + N)
    x = (torch.randn(R, K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16)
    ap, an = float(pz.softplus(0.4)), 0.5 + float(pz.softplus(-0.3))
    ref = pz.xielu(x.double().numpy() @ w.double().numpy().T, 0.4, -0.3)
    out = ops().linear_xielu(x.to(DEV), w.to(DEV), ap, an)
    assert out.dtype == torch.bfloat16 and relerr(out, ref) < 1.2e-2
    x32, w32 = x.float(), w.float()
    assert relerr(ops().linear_xielu(x32.to(DEV), w32.to(DEV), ap, an), ref) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,dv,rot,col0,extra", [
    (4, 2, 16, 24, (100.0, 8), 0, 64), (3, 3, 40, 16, (1000.0, 20), 8, 120), (8, 2, 128, 64, (500000.0, 32), 0, 0),
    (2, 1, 64, 32, (10000.0, 64), 16, 128), (6, 1, 8, 8, None, 0, 5), (12, 3, 32, 128, (10000.0, 16), 4, 0)])
def test_partial_rotation_and_the_cache_write_with_values_of_another_size(dtype, nq, nkv, d, dv, rot, col0, extra):
    """Rows of a stacked product [other columns | q | k | v | further columns]: q and
    k rotated on their first dimensions; keys and values into pages of their own
    widths.  Positions far out (large angles), at a page's edge and at zero."""
    from reflex_b200.config.spec import PositionSpec
    from reflex_b200.parts.registry import POSITIONS

    g = torch.Generator().manual_seed(nq + d)
    pos = [0, 1, 63, 64, 65, 1000, 4099]
    R = len(pos)
    ld = (nq + nkv) * d + nkv * dv
    proj = torch.randn(R, col0 + ld + extra, generator=g) * 2
    rotation = None
    if rot is not None:
        spec = PositionSpec("rope_neox", d, rot[1], rot[0])
        rotation = POSITIONS.get(spec.kind)(spec, dtype, DEV).rotation()
    n_pages = 4099 // 64 + 1
    table = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, n_pages).contiguous()
    kp = torch.zeros(n_pages, nkv, 64, d, dtype=dtype, device=DEV)
    vp = torch.zeros(n_pages, nkv, 64, dv, dtype=dtype, device=DEV)
    q = ops().sig_qkv_post(proj.to(DEV), col0, rotation, i32(pos), i32([0] * R), kp, vp, table.to(DEV), 64, nq, nkv,
                           d, dv, True, dtype)
    x = proj.double().numpy()[:, col0:]
    dims, base = (rot[1], rot[0]) if rot else (0, 1.0)
    qr = pz.rotate(x[:, :nq * d].reshape(R, nq, d), np.array(pos), dims, base)
    kr = pz.rotate(x[:, nq * d:(nq + nkv) * d].reshape(R, nkv, d), np.array(pos), dims, base)
    vr = x[:, (nq + nkv) * d:ld].reshape(R, nkv, dv)
    # 32-bit angles: at position 4,099 an angle of thousands of radians is known to a few 1e-4 of one
    t = 3e-4 if dtype == torch.float32 else 8e-3
    assert relerr(q.reshape(R, nq, d), qr) < t
    for r, p in enumerate(pos):
        page = int(table[0, p // 64])
        assert relerr(kp[page, :, p % 64], kr[r]) < t, p
        assert relerr(vp[page, :, p % 64], vr[r]) < (1e-7 if dtype == torch.float32 else 8e-3), p


def _paged_kv(seqs, nkv, d, dv, dtype, g, fill=float("nan")):
    """Random keys and values for sequences of the given total lengths in a scrambled
    paged store whose unused rows hold `fill` (NaN: reading one shows)."""
    per = [(n + 63) // 64 for n in seqs]
    total = sum(per) + 5
    perm = torch.randperm(total, generator=g)
    table = torch.full((len(seqs) + 3, max(per) + 2), -12345, dtype=torch.int32)
    slots = torch.randperm(len(seqs) + 3, generator=g)[: len(seqs)].tolist()
    k_pages = torch.full((total, nkv, 64, d), fill, dtype=torch.float32)
    v_pages = torch.full((total, nkv, 64, dv), fill, dtype=torch.float32)
    ks, vs, o = [], [], 0
    for i, n in enumerate(seqs):
        k, v = torch.randn(n, nkv, d, generator=g), torch.randn(n, nkv, dv, generator=g)
        for p in range(per[i]):
            page = int(perm[o + p])
            table[slots[i], p] = page
            m = min(64, n - p * 64)
            k_pages[page, :, :m] = k[p * 64:p * 64 + m].transpose(0, 1)
            v_pages[page, :, :m] = v[p * 64:p * 64 + m].transpose(0, 1)
        o += per[i]
        ks.append(k)
        vs.append(v)
    return slots, table, k_pages.to(dtype), v_pages.to(dtype), ks, vs


def _sigmoid_ref(q, ks, vs, seqs, scale, window, bias, dtype):
    outs, r = [], 0
    for (start, n), k, v in zip(seqs, ks, vs):
        kk, vv = k.to(dtype).double().numpy(), v.to(dtype).double().numpy()
        for t in range(n):
            i = start + t
            lo = max(0, i - window + 1) if window else 0
            o = np.zeros((q.shape[1], vv.shape[2]))
            for h in range(q.shape[1]):
                kvh = h // (q.shape[1] // kk.shape[1])
                s = (kk[lo:i + 1, kvh] @ q[r + t, h].to(dtype).double().numpy()) * scale + bias[h]
                o[h] = (pz.sigmoid(s)[:, None] * vv[lo:i + 1, kvh]).sum(0)
            outs.append(o)
        r += n
    return np.stack(outs)


SIG_CASES = [  # nq, nkv, d, dv, [(start, n_new)], window
    (4, 2, 16, 24, [(0, 70), (130, 3), (0, 1)], 20),
    (2, 1, 64, 32, [(0, 200), (63, 2), (133, 3)], 70),
    (6, 2, 64, 128, [(0, 300), (328, 4)], 150),
    (8, 2, 128, 64, [(0, 150), (200, 40)], 33),
    (3, 3, 40, 16, [(0, 140)], 64),                   # a window of exactly a page
    (12, 3, 32, 128, [(0, 260), (5, 1)], None),       # every earlier key
    (6, 1, 8, 8, [(0, 5), (64, 1), (127, 2)], 1),     # a window of one: the token itself
    (16, 1, 64, 64, [(500, 1), (63, 1), (64, 1), (0, 1)], 200),   # a row a sequence: decoding
]
SIG_KERNELS = ["plain_f32", "plain_bf16", "mma_bf16"]


@pytest.mark.parametrize("kernel", SIG_KERNELS)
@pytest.mark.parametrize("nq,nkv,d,dv,seqs,window", SIG_CASES)
def test_sigmoid_weights_over_a_window_in_every_attention_kernel(kernel, nq, nkv, d, dv, seqs, window):
    dtype = torch.float32 if kernel.endswith("f32") else torch.bfloat16
    g = torch.Generator().manual_seed(nq * 100 + d)
    totals = [s + n for s, n in seqs]
    slots, table, kp, vp, ks, vs = _paged_kv(totals, nkv, d, dv, dtype, g)
    R = sum(n for _, n in seqs)
    q = torch.randn(R, nq, d, generator=g)
    bias = (torch.randn(nq, generator=g) * 2 - 1).double().numpy()
    scale = 1.5 / math.sqrt(d)
    cut = [(k[:s + n], v[:s + n]) for (s, n), k, v in zip(seqs, ks, vs)]
    ref = _sigmoid_ref(q, [c[0] for c in cut], [c[1] for c in cut], seqs, scale, window, bias, dtype)
    batch = FakeBatch([[0] * n for _, n in seqs], slots, [s for s, _ in seqs])
    batch.is_decode = all(n == 1 for _, n in seqs)
    batch.max_new = max(n for _, n in seqs)
    batch.max_context = max(totals)
    qd = q.to(dtype).reshape(R, nq * d).to(DEV)
    args = (qd, kp.to(DEV), vp.to(DEV), table.to(DEV), 64)
    if kernel.startswith("plain"):
        out = ops().attention_sigmoid_plain(*args, batch.row_pos, batch.row_slot, nq, nkv, d, dv, window, scale,
                                            f32(bias))
    else:
        out = ops().attention_sigmoid_mma(*args, batch.seq_slot, batch.seq_start, batch.seq_new, batch.seq_row0,
                                          batch.max_new, nq, nkv, d, dv, window, scale, f32(bias))
    assert relerr(out.reshape(R, nq, dv), ref) < tol(dtype, 2e-5, 1.5e-2)


@pytest.mark.parametrize("kernel", SIG_KERNELS)
@pytest.mark.parametrize("steps", ["prompt", "decode"])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_window(kernel, steps):
    """Every key weighs next to nothing (a bias of -12) but one, at position 100,
    whose score is large: queries up to position 100 + window - 1 find its value,
    the next one does not.  A window that is one token off shows as a whole value."""
    dtype = torch.float32 if kernel.endswith("f32") else torch.bfloat16
    nq, nkv, d, dv, window, T = 4, 2, 32, 48, 77, 260
    g = torch.Generator().manual_seed(9)
    k = torch.randn(T, nkv, d, generator=g) * 0.05
    v = torch.randn(T, nkv, dv, generator=g)
    k[100] = 0.0
    k[100, :, 3] = 8.0
    v[100] = 50.0
    q = torch.randn(T, nq, d, generator=g) * 0.05
    q[:, :, 3] = 4.0     # 32 against the one key, about zero against the others
    n_pages = (T + 63) // 64
    table = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, n_pages).contiguous()
    kp = torch.zeros(n_pages, nkv, 64, d)
    vp = torch.zeros(n_pages, nkv, 64, dv)
    for p in range(T):
        kp[int(table[0, p // 64]), :, p % 64] = k[p]
        vp[int(table[0, p // 64]), :, p % 64] = v[p]
    bias = f32([-12.0] * nq)
    seen = {}
    for i in (99, 100, 101, 100 + window - 2, 100 + window - 1, 100 + window, 100 + window + 1, T - 1):
        if steps == "prompt":
            start, n = max(0, i - 40), min(i, 40) + 1   # the query is the last row of a portion
        else:
            start, n = i, 1
        batch = FakeBatch([[0] * n], [0], [start])
        batch.is_decode, batch.max_new, batch.max_context = n == 1, n, start + n
        qd = q[start:start + n].to(dtype).reshape(n, nq * d).to(DEV)
        args = (qd, kp.to(dtype).to(DEV), vp.to(dtype).to(DEV), table.to(DEV), 64)
        if kernel.startswith("plain"):
            out = ops().attention_sigmoid_plain(*args, batch.row_pos, batch.row_slot, nq, nkv, d, dv, window, 1.0, bias)
        else:
            out = ops().attention_sigmoid_mma(*args, batch.seq_slot, batch.seq_start, batch.seq_new, batch.seq_row0,
                                              batch.max_new, nq, nkv, d, dv, window, 1.0, bias)
        seen[i] = float(out.float().reshape(n, nq, dv)[-1].abs().max())
    for i, m in seen.items():
        inside = 100 <= i <= 100 + window - 1
        assert (m > 45.0) == inside and (inside or m < 1.0), (i, m)


def _ssd_ref(proj, w, m, eps):
    """The mixer's gated, normed y for whole sequences, from the in product's rows."""
    T = proj.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = pz.silu(pz.causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, Hh, P)
    B, C = xbc[:, inner:inner + G * N].reshape(T, G, N), xbc[:, inner + G * N:].reshape(T, G, N)
    y = pz.ssd_scan(x, B, C, pz.softplus(dt + w["dt_bias"]), -np.exp(w["A_log"]), w["D"], Hh, G).reshape(T, inner)
    y = y * pz.silu(z)
    return pz.rms_unit(y.reshape(T, m["norm_groups"], -1), eps).reshape(T, inner) * w["norm"]


@pytest.mark.parametrize("heads,P,N,G,taps,parts", [(2, 16, 8, 1, 3, 1), (3, 24, 1, 3, 1, 1), (2, 48, 40, 2, 5, 2),
                                                    (8, 64, 64, 2, 4, 2), (6, 16, 24, 3, 2, 3), (4, 8, 16, 2, 4, 4),
                                                    (1, 33, 130, 1, 2, 1)])
@pytest.mark.parametrize("gap", [1, 4])
def test_filter_and_state_space_scan_carried_through_their_state(heads, P, N, G, taps, parts, gap):
    """Two sequences side by side in slots of a state tensor that held other numbers
    before: whole, and in steps down to one and two rows (fewer than the filter
    looks back)."""
    from reflex_b200.config.spec import MixerSpec
    from reflex_b200.parts.ssd import StateSpaceDuality

    g = torch.Generator().manual_seed(heads * 10 + N)
    inner, cc = heads * P, heads * P + 2 * G * N
    m = {"heads": heads, "vdim": P, "state": N, "groups": G, "norm_groups": parts}
    spec = MixerSpec("ssd", hidden_size=32, params=(("heads", heads), ("vdim", P), ("state", N), ("groups", G),
                                                    ("taps", taps), ("norm_groups", parts), ("eps", 1e-5)))
    part = StateSpaceDuality(spec, torch.float32, DEV)
    w = {"conv": torch.rand(cc, taps, generator=g) * 1.2 - 0.6, "conv.b": torch.rand(cc, generator=g) - 0.5,
         "dt_bias": torch.rand(heads, generator=g) * 2 - 1, "A_log": torch.rand(heads, generator=g) * 2 - 1.5,
         "D": torch.rand(heads, generator=g) - 0.5, "norm": torch.rand(inner, generator=g) + 0.5}
    part.bind({"in_proj": torch.zeros(inner + cc + heads, 32), "conv": w["conv"], "conv_bias": w["conv.b"],
               "dt_bias": w["dt_bias"], "A_log": w["A_log"], "D": w["D"], "norm": w["norm"],
               "o_proj": torch.zeros(32, inner)})
    wn = {k: v.double().numpy() for k, v in w.items()}
    lens = [37, 70]
    projs = [torch.randn(n, 7 + inner + cc + heads, generator=g) * 1.5 for n in lens]
    refs = [_ssd_ref(p.double().numpy()[:, 7:], wn, m, 1e-5) for p in projs]

    class Ctx:
        pass

    for cuts in ([100], [gap], [5, 1, 2, 33]):
        state = torch.randn(5, part.cache_spec().shape[0], generator=g).to(DEV)  # slots used before
        state[1].zero_()
        state[3].zero_()
        fed, got, step = [0, 0], [[], []], 0
        while any(f < n for f, n in zip(fed, lens)):
            take = [min(cuts[min(step, len(cuts) - 1)], n - f) for f, n in zip(fed, lens)]
            live = [i for i in range(2) if take[i] > 0]
            ctx = Ctx()
            ctx.batch = FakeBatch([[0] * take[i] for i in live], [[3, 1][i] for i in live], [fed[i] for i in live])
            ctx.state = state
            rows = torch.cat([projs[i][fed[i]:fed[i] + take[i]] for i in live]).to(DEV).contiguous()
            y = part.normed_out(None, ctx, proj=(rows, 7)).cpu().double().numpy()
            r = 0
            for i in live:
                got[i].append(y[r:r + take[i]])
                r += take[i]
                fed[i] += take[i]
            step += 1
        for i in range(2):
            assert relerr(np.concatenate(got[i]), refs[i]) < 3e-5, (cuts, i)


@pytest.mark.parametrize("heads,d,rank", [(2, 16, 4), (1, 32, 8), (5, 20, 3), (2, 128, 16), (3, 8, 1), (2, 50, 5),
                                          (1, 64, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_delta_rule_carried_through_its_state(heads, d, rank, dtype):
    """The mixer without its output product, two sequences in reused slots: whole,
    token by token, and in unequal steps."""
    from reflex_b200.config.spec import MixerSpec
    from reflex_b200.parts.delta_rule import DeltaRule

    g = torch.Generator().manual_seed(heads * 10 + d)
    W, hd = 40, heads * d
    spec = MixerSpec("delta_rule", hidden_size=W, num_heads=heads, head_dim=d,
                     params=(("rate", math.exp(-0.5)), ("unit_eps", 1e-6), ("eps", 1e-5)))
    part = DeltaRule(spec, dtype, DEV)
    t = {"r_proj": torch.randn(hd, W, generator=g) * 0.3, "k_proj": torch.randn(hd, W, generator=g) * 0.5,
         "v_proj": torch.randn(hd, W, generator=g) * 0.3, "g_proj": torch.randn(hd, W, generator=g) * 0.3,
         "a_proj": torch.randn(hd, W, generator=g) * 0.3, "a_bias": torch.rand(hd, generator=g) - 0.5,
         "w1_proj": torch.randn(rank, W, generator=g) * 0.3, "w2_proj": torch.randn(hd, rank, generator=g),
         "w0": torch.rand(hd, generator=g) - 0.5, "norm": torch.rand(hd, generator=g) + 0.5,
         "o_proj": torch.eye(hd)}   # the output product passes the heads through
    t = {k: v.to(dtype).float() for k, v in t.items()}      # what both sides see
    part.bind(dict(t))
    names = {"r_proj": "r", "k_proj": "k", "v_proj": "v", "g_proj": "g", "a_proj": "a", "a_bias": "a.b",
             "w1_proj": "w1", "w2_proj": "w2", "w0": "w0", "norm": "norm", "o_proj": "o"}
    wn = {names[k]: v.double().numpy() for k, v in t.items()}
    lens = [45, 80]
    xs = [torch.randn(n, W, generator=g).to(dtype).float() for n in lens]
    refs = [pz.delta_mixer(x.double().numpy(), wn, {"heads": heads, "dim": d}, 1e-5) for x in xs]

    class Ctx:
        pass

    for cuts in ([100], [1], [7, 2, 1, 40]):
        state = torch.randn(4, heads * d * d, generator=g).to(DEV)
        state[0].zero_()
        state[2].zero_()
        fed, got, step = [0, 0], [[], []], 0
        while any(f < n for f, n in zip(fed, lens)):
            take = [min(cuts[min(step, len(cuts) - 1)], n - f) for f, n in zip(fed, lens)]
            live = [i for i in range(2) if take[i] > 0]
            ctx = Ctx()
            ctx.batch = FakeBatch([[0] * take[i] for i in live], [[2, 0][i] for i in live], [fed[i] for i in live])
            ctx.state = state
            rows = torch.cat([xs[i][fed[i]:fed[i] + take[i]] for i in live]).to(dtype).to(DEV).contiguous()
            y = part.forward(rows, ctx).cpu().double().numpy()
            r = 0
            for i in live:
                got[i].append(y[r:r + take[i]])
                r += take[i]
                fed[i] += take[i]
            step += 1
        for i in range(2):
            assert relerr(np.concatenate(got[i]), refs[i]) < tol(dtype, 5e-5, 3e-2), (cuts, i)


def test_a_slow_decay_keeps_a_far_input_and_a_removal_rate_of_one_forgets_it():
    """Delta rule, one head: with decays near one and no removal a value written at the
    first token is read 300 tokens later; with a removal rate of one along the same key
    it is gone after the second token."""
    heads, d, T = 1, 16, 300
    hd = heads * d
    k = np.zeros((T, hd))
    k[:, 0] = 1.0
    v = np.zeros((T, hd))
    v[0, 5] = 7.0
    r = np.zeros((T, hd))
    r[:, 0] = 1.0
    for a_pre, w_pre, want in ((-40.0, -40.0, 7.0), (40.0, -40.0, 0.0)):
        proj = np.concatenate([r, k, v, np.full((T, hd), a_pre)], axis=1)
        state = torch.zeros(1, hd * d, device=DEV)
        batch = FakeBatch([[0] * T], [0], [0])
        o = ops().delta_rule(f32(proj), 0, hd, 2 * hd, 3 * hd, f32(np.full((T, hd), w_pre)), f32(np.zeros(hd)),
                             f32(np.zeros(hd)), math.exp(-0.5), 1e-6, state, 0, batch, heads, d).cpu().numpy()
        assert abs(o[0, 5] - 7.0) < 1e-5 and abs(o[-1, 5] - want) < 1e-4, (a_pre, o[1, 5], o[-1, 5])


@pytest.mark.parametrize("R", [1, 2, 5, 9, 70, 200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,scale,shared", [(8, 3, 1.25, 64), (4, 2, 1.0, 0), (1, 1, 2.0, 16), (3, 3, 0.5, 0)])
def test_experts_with_scores_over_all_of_them_and_a_shared_expert(R, dtype, E, top, scale, shared):
    from reflex_b200.config.spec import FeedForwardSpec
    from reflex_b200.parts.moe import MixtureOfExperts

    g = torch.Generator().manual_seed(R * 7 + E)
    W, ff = 64, 24
    spec = FeedForwardSpec("moe", hidden_size=W, intermediate_size=ff, params=(
        ("experts", E), ("top", top), ("activation", "swiglu"), ("scores", "softmax_all"), ("score_scale", scale),
        ("shared_ff", shared), ("shared_kind", "swiglu")))
    part = MixtureOfExperts(spec, dtype, DEV)
    t = {"router": torch.randn(E, W, generator=g) * 0.5}
    for e in range(E):
        t[f"expert_gate#{e}"] = torch.randn(ff, W, generator=g) * 0.2
        t[f"expert_up#{e}"] = torch.randn(ff, W, generator=g) * 0.2
        t[f"expert_down#{e}"] = torch.randn(W, ff, generator=g) * 0.2
    if shared:
        t.update({"shared_gate": torch.randn(shared, W, generator=g) * 0.2, "shared_up": torch.randn(shared, W, generator=g) * 0.2,
                  "shared_down": torch.randn(W, shared, generator=g) * 0.2})
    t = {k: v.to(dtype).float() for k, v in t.items()}
    part.bind(dict(t))
    wn = {"router": t["router"].double().numpy()}
    for e in range(E):
        for n in ("gate", "up", "down"):
            wn[f"e{e}.{n}"] = t[f"expert_{n}#{e}"].double().numpy()
    for n in ("gate", "up", "down"):
        if shared:
            wn[f"shared.{n}"] = t[f"shared_{n}"].double().numpy()
    x = torch.randn(R, W, generator=g).to(dtype).float()
    mlp = {"router": {"experts": E, "top": top, "scale": scale}, "shared": {"ff": shared} if shared else None}
    ref = pz.moe_ff(x.double().numpy(), wn, mlp)
    out = part.forward(x.to(dtype).to(DEV))
    assert relerr(out, ref) < tol(dtype, 1e-5, 2.5e-2)


def test_routing_weights_and_ties():
    logits = torch.tensor([[0.0, 2.0, 2.0, -1.0, 1.0], [5.0, 5.0, 5.0, 5.0, 5.0], [-30.0, 40.0, 0.0, 39.0, 1.0]])
    ids, wts = ops().moe_route(logits.to(DEV), None, 3, scores="softmax_all", scale=1.25)
    assert ids.cpu().tolist() == [[1, 2, 4], [0, 1, 2], [1, 3, 4]]   # ties: the lower index
    _ids, ref = pz.route(logits.double().numpy(), np.eye(5), 3, 1.25)
    assert relerr(wts, ref) < 1e-6 and abs(float(wts[1].sum()) - 1.25) < 1e-6


# ----------------------------------------------------------------- whole models
def sharpness(dtype):
    """The full factors in 32-bit; their square roots in bfloat16 (`zelinex_models.model_folder`)."""
    return True if dtype in ("float32", "f32") else "mild"


def make_engine(name, dtype, max_tokens=4096, **kw):
    import reflex_b200
    from reflex_b200.engine import Engine

    model = reflex_b200.load_model(zm.model_folder(name, sharp=sharpness(dtype)), dtype, DEV)
    return Engine(model, max_tokens=max_tokens, **kw)


_PLAIN = {}


def plain_logits(name, toks, dtype="float32"):
    key = (name, tuple(toks), sharpness(dtype))
    if key not in _PLAIN:
        cfg, w = pz.read_model(zm.model_folder(name, sharp=sharpness(dtype)))
        _PLAIN[key] = pz.forward(cfg, w, toks)
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
    """The residual after every layer run of a looped model, 32-bit."""
    eng = make_engine(name, "float32")
    model = eng.model
    toks = zm.tokens(40, zm.ALL[name]["vocab"], 3)
    cfg, w = pz.read_model(zm.model_folder(name))
    ref = []
    pz.forward(cfg, w, toks, layers_out=ref)
    seen = []

    def after(i, run, layer, h, pending):
        seen.append(h.cpu().double().numpy().copy())

    model.after_run = after
    s = eng.open()
    eng.step([(s, toks, [0])])
    eng.close(s)
    model.after_run = None
    assert len(seen) == len(ref) == 5
    for i, (a, b) in enumerate(zip(seen, ref)):
        assert np.abs(a - b).max() / np.abs(b).max() < 5e-5, (i, np.abs(a - b).max() / np.abs(b).max())


@pytest.mark.parametrize("name", sorted(zm.ALL))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_token_by_token_equal_the_plain_model(name, dtype):
    """Each position's logits, with the prompt in one step, token by token from
    the very first token, and in portions of several sizes down to two tokens:
    the windows' edges, the filters' look back, every page's edge and the first
    tokens are met both inside a prompt and in decoding."""
    eng = make_engine(name, dtype)
    toks = zm.tokens(LENGTHS[name], zm.ALL[name]["vocab"], 11)
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
    vocab = zm.ALL[name]["vocab"]
    lens = [1, 70, 3, 131, 64, 9, 200, 2]
    reqs = [zm.tokens(n, vocab, 20 + i) for i, n in enumerate(lens)]
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
    """A short prompt and 500 decoded tokens: the recurrences' states and the filter's
    last inputs are carried for hundreds of steps, both windows pass over decoded
    tokens many times and their pages are given back."""
    eng = make_engine("A", dtype, max_tokens=1024)
    toks = zm.tokens(510, zm.ALL["A"]["vocab"], 5)
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
    folder = zm.model_folder(name, sharp=sharpness(dtype))
    model = reflex_b200.Model.load(folder, weights=dtype, max_tokens=2048, max_batch=3)
    vocab = zm.ALL[name]["vocab"]
    prompts = [zm.tokens(n, vocab, 40 + n) for n in (5, 70, 1, 130)]
    n_new = 12
    got = model.generate(prompts, n_new)
    cfg, w = pz.read_model(folder)
    for p, out in zip(prompts, got):
        assert len(out) == n_new
        seq = list(p)
        for t, tok in enumerate(out):
            lg = pz.forward(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if dtype == "bf16" and top2[1] - top2[0] < 0.15 * np.abs(lg).max():
                break  # a near tie: bfloat16 may pick the other one, and the continuations part
            assert tok == int(np.flatnonzero(lg == lg.max())[-1]), (len(p), t)
            seq.append(tok)


def test_decode_steps_are_captured_into_graphs():
    eng = make_engine("E", "bfloat16")
    assert eng.model.capturable and eng.use_graphs
