// Selective scan (a diagonal state-space recurrence with input-dependent steps).
//
// For channel c and state index n, token by token through a sequence:
//     dt_c   = softplus(dtpre[t][c] + dt_bias[c])
//     S[c,n] <- exp(dt_c * A[c,n]) * S[c,n] + dt_c * x[t][c] * B[t][n]
//     y_c    = sum_n S[c,n] * C[t][n] + D[c] * x[t][c]
//     out    = y_c * silu(z[t][c])
// with A = -exp(A_log) made once when the weights are bound.  S is the
// sequence's state, [channels][N] 32-bit floats in its slot of the cache's
// state group (zero when the slot is taken), read when a step begins and
// written when it ends, so the recurrence goes on however the tokens were cut.
// Everything here is 32-bit: the step sizes, the decays' exponentials, the
// state, the sums; only `out` takes the product's type.
//
// Work layout: LPC neighbouring lanes share a channel, lane j of them holds
// states j, j + LPC, ... (NPL of them, in registers); a token costs each lane
// NPL exponentials and 2 NPL multiply-adds, and the lanes' partial y meet by
// shuffles.  A block takes 128 / LPC channels of one sequence and walks its rows
// in order; the next row's operands are loaded while this row's chain runs.
// That form serves steps of a row or two a sequence (decoding).
//
// Prompts take the tiled, segmented form.  A lane holds up to 16 states of a
// channel (one lane a channel up to 16 states: no shuffles, sixteen independent
// chains a row), and since that leaves few threads, a sequence's rows are cut
// into G segments that run side by side.  The recurrence is linear in S, so
//   (1) every segment but the last folds its rows from S = 0 into S_local and
//       the sum of its step sizes (the segment's decay is exp(A * that sum)),
//   (2) a small kernel carries the sequence's state through the segments,
//       S_begin[g + 1] = exp(A * sum_dt[g]) * S_begin[g] + S_local[g],
//   (3) every segment runs again from its S_begin and writes its rows; the last
//       one leaves the sequence's state.
// With G = 1 only (3) runs, from the state.  A block walks its segment in tiles
// of TT rows whose operands (its channels' x, dt and z, the rows' B and C) arrive
// in shared memory by asynchronous copies while the tile before is computed, so
// a step of the recurrence waits for no load.  Per tile: (A) every thread turns
// some of the tile's dt into softplus(dt + bias) and z into silu(z), each once a
// channel; (B) the recurrence; (C) the tile's results leave in row order.
// The decay of a step is 2^(dt * A * log2 e) in every form, A * log2 e made when
// the block starts.
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int THREADS = 128;

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }
// 2^v for v <= 0 (a decay): the hardware's base-2 exponential, results below 2^-126 are zero
__device__ __forceinline__ float decay2(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

// The step size's last product inside the row-by-row form: channel c's row of W_dt
// ([channels][rank], bfloat16 or 32-bit) times the row's low-rank vector, shared by the
// channel's lanes and met by shuffles.  With bfloat16 weights the vector is rounded to
// bfloat16 first, as the product kernel's input would be.
struct StepRank {
    const void* w;     // null: the step sizes come ready in `dtpre`
    int bf16;          // the weights' type
    int rank;
    int off;           // the vector's first column in the B | C rows
};

__device__ __forceinline__ float step_from_rank(const StepRank& sr, int c, const float* __restrict__ low, int sub,
                                                int lpc) {
    float acc = 0.0f;
    if (sr.bf16) {
        const __nv_bfloat16* wr = reinterpret_cast<const __nv_bfloat16*>(sr.w) + (size_t)c * sr.rank;
#pragma unroll 4
        for (int j = sub; j < sr.rank; j += lpc)
            acc = fmaf(__bfloat162float(wr[j]), __bfloat162float(__float2bfloat16_rn(low[j])), acc);
    } else {
        const float* wr = reinterpret_cast<const float*>(sr.w) + (size_t)c * sr.rank;
#pragma unroll 4
        for (int j = sub; j < sr.rank; j += lpc) acc = fmaf(wr[j], low[j], acc);
    }
    for (int o = lpc >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    return acc;
}

template <typename TO, int NPL>
__global__ void __launch_bounds__(THREADS)
mamba_scan_kernel(const float* __restrict__ x, const float* __restrict__ dtpre, const float* __restrict__ dt_bias,
                  const float* __restrict__ bc, int ld_bc, int b_off, int c_off,
                  const float* __restrict__ zsrc, int ld_z, int z_off, const float* __restrict__ A,
                  const float* __restrict__ Dw, float* __restrict__ state, size_t slot_stride, size_t state_off,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_row0, TO* __restrict__ out,
                  int channels, int N, int lpc, StepRank sr) {
    pdl_launch_dependents();
    const int s = blockIdx.x;
    const int sub = threadIdx.x % lpc;                       // which share of the channel's states
    const int c = blockIdx.y * (THREADS / lpc) + threadIdx.x / lpc;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;                  // lanes beyond the end follow along and store nothing
    // the weights: no kernel writes them
    float a[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int n = sub + i * lpc;
        a[i] = n < N ? A[(size_t)cc * N + n] * LOG2E : 0.0f;
    }
    const float bias = dt_bias ? dt_bias[cc] : 0.0f;
    const float d_skip = Dw ? Dw[cc] : 0.0f;
    pdl_wait();
    const int row0 = seq_row0[s], rows = seq_row0[s + 1] - row0;
    float* st_c = state + (size_t)seq_slot[s] * slot_stride + state_off + (size_t)cc * N;
    float S[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int n = sub + i * lpc;
        S[i] = n < N ? st_c[n] : 0.0f;
    }
    // the operands of row t: this channel's x, dt and z, the row's B and C
    float xv, dv, zv, Bv[NPL], Cv[NPL];
    auto fetch = [&](int t) {
        const size_t r = (size_t)(row0 + t);
        xv = x[r * channels + cc];
        zv = zsrc[r * ld_z + z_off + cc];
        const float* brow = bc + r * ld_bc;
        dv = sr.w ? step_from_rank(sr, cc, brow + sr.off, sub, lpc) : dtpre[r * channels + cc];
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int n = sub + i * lpc;
            Bv[i] = n < N ? brow[b_off + n] : 0.0f;
            Cv[i] = n < N ? brow[c_off + n] : 0.0f;
        }
    };
    if (rows > 0) fetch(0);
#pragma unroll 1
    for (int t = 0; t < rows; ++t) {
        const float xt = xv, zt = zv;
        const float dt = softplus_f(dv + bias);
        float Bt[NPL], Ct[NPL];
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            Bt[i] = Bv[i];
            Ct[i] = Cv[i];
        }
        if (t + 1 < rows) fetch(t + 1);
        const float dx = dt * xt;
        float y = 0.0f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            S[i] = fmaf(decay2(dt * a[i]), S[i], dx * Bt[i]);
            y = fmaf(S[i], Ct[i], y);
        }
        for (int o = lpc >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (sub == 0 && live) {
            y = fmaf(d_skip, xt, y);
            const float g = zt / (1.0f + expf(-zt));
            rfx::st<TO>(out, (size_t)(row0 + t) * channels + c, y * g);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int n = sub + i * lpc;
            if (n < N) st_c[n] = S[i];
        }
    }
}


// ------------------------------------------------------- tiled, segmented form
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int K> __device__ __forceinline__ void copy_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory");
}

// segment g of G of a sequence of `rows` rows: [begin, begin + count)
__device__ __forceinline__ void segment_of(int rows, int G, int g, int& begin, int& count) {
    const int L = (rows + G - 1) / G;
    begin = min(rows, g * L);
    count = min(rows, begin + L) - begin;
}

// How the threads of a block share its work, the same for all three kernels.
struct ScanPlan {
    int lpc;       // lanes a channel (a power of two), lane j holds states j * NPL ...
    int lp_shift;  // log2(lpc)
    int ch_shift;  // log2(channels of a block) = log2(THREADS / lpc)
    int TT;        // rows a tile
    int G;         // segments a sequence
};

// softplus and silu of a (row, channel), once a tile.  FAST (results that are rounded to
// bfloat16): the hardware's exponential, logarithm and division, about 1e-6 of the value.
template <bool FAST> __device__ __forceinline__ float softplus_t(float v) {
    if constexpr (FAST) {
        const float e = __expf(-fabsf(v));
        return fmaxf(v, 0.0f) + (e < 1e-4f ? e : __logf(1.0f + e));
    }
    return softplus_f(v);
}
template <bool FAST> __device__ __forceinline__ float silu_t(float z) {
    if constexpr (FAST) return __fdividef(z, 1.0f + __expf(-z));
    return z / (1.0f + expf(-z));
}

// V floats a copy: 4 where every address involved is a multiple of 16 bytes, else 1.
// FOLD: step (1), no output; else step (3).  FAST: see above; both steps of a scan take the same.
template <typename TO, int NPL, int V, bool FOLD, bool FAST>
__global__ void __launch_bounds__(THREADS)
mamba_scan_tiled_kernel(const float* __restrict__ x, const float* __restrict__ dtpre,
                        const float* __restrict__ dt_bias, const float* __restrict__ bc, int ld_bc, int b_off,
                        int c_off, const float* __restrict__ zsrc, int ld_z, int z_off,
                        const float* __restrict__ A, const float* __restrict__ Dw, float* __restrict__ state,
                        size_t slot_stride, size_t state_off, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_row0, TO* __restrict__ out, int channels, int N,
                        ScanPlan plan, float* __restrict__ seg_local, float* __restrict__ seg_dt,
                        const float* __restrict__ seg_begin) {
    extern __shared__ float4 tiles4[];
    float* tiles = reinterpret_cast<float*>(tiles4);
    pdl_launch_dependents();
    const int G = plan.G, g = blockIdx.z;
    if (FOLD && g == G - 1) return;  // the last segment's fold is nobody's input
    const int TT = plan.TT;
    const int CH = 1 << plan.ch_shift;
    const int stage_floats = TT * (3 * CH + 2 * N);
    const int s = blockIdx.x;
    const int c0 = blockIdx.y * CH;
    const int lc = threadIdx.x >> plan.lp_shift, sub = threadIdx.x & (plan.lpc - 1);
    const int c = c0 + lc;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;
    const int n0 = sub * NPL;
    float a2[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) a2[i] = n0 + i < N ? A[(size_t)cc * N + n0 + i] * LOG2E : 0.0f;
    const float d_skip = (!FOLD && Dw) ? Dw[cc] : 0.0f;
    pdl_wait();
    const int row0 = seq_row0[s], rows = seq_row0[s + 1] - row0;
    int seg0, count;
    segment_of(rows, G, g, seg0, count);
    const size_t seg_cell = ((size_t)s * G + g) * channels + cc;  // this channel's place in the segments' arrays
    float* st_c = state + (size_t)seq_slot[s] * slot_stride + state_off + (size_t)cc * N;
    float S[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        if (FOLD || n0 + i >= N) S[i] = 0.0f;
        else S[i] = G == 1 ? st_c[n0 + i] : seg_begin[seg_cell * N + n0 + i];
    }
    float sum_dt = 0.0f;
    const int ntiles = (count + TT - 1) / TT;
    auto load = [&](int k, int st) {
        float* xs = tiles + (size_t)st * stage_floats;
        float* ds = xs + TT * CH;
        float* zs = ds + TT * CH;
        float* bs = zs + TT * CH;
        float* cs = bs + TT * N;
        const int t_begin = seg0 + k * TT;
        const int valid = min(TT, seg0 + count - t_begin);
        for (int i = threadIdx.x * V; i < valid * CH; i += THREADS * V) {
            const int t = i >> plan.ch_shift, l = i & (CH - 1);
            if (c0 + l >= channels) continue;
            const size_t r = (size_t)(row0 + t_begin + t);
            if (V == 4) {
                copy_async16(xs + i, x + r * channels + c0 + l);
                copy_async16(ds + i, dtpre + r * channels + c0 + l);
                if (!FOLD) copy_async16(zs + i, zsrc + r * ld_z + z_off + c0 + l);
            } else {
                copy_async4(xs + i, x + r * channels + c0 + l);
                copy_async4(ds + i, dtpre + r * channels + c0 + l);
                if (!FOLD) copy_async4(zs + i, zsrc + r * ld_z + z_off + c0 + l);
            }
        }
        for (int i = threadIdx.x * V; i < valid * N; i += THREADS * V) {
            const int t = i / N, n = i - t * N;
            const float* brow = bc + (size_t)(row0 + t_begin + t) * ld_bc;
            if (V == 4) {
                copy_async16(bs + i, brow + b_off + n);
                if (!FOLD) copy_async16(cs + i, brow + c_off + n);
            } else {
                copy_async4(bs + i, brow + b_off + n);
                if (!FOLD) copy_async4(cs + i, brow + c_off + n);
            }
        }
    };
    if (ntiles > 0) load(0, 0);
    copy_commit();
    const int mine = c0 + (threadIdx.x & (CH - 1));  // the channel of this thread's share of (A)
    const bool mine_live = mine < channels;
    const float mine_bias = (dt_bias && mine_live) ? dt_bias[mine] : 0.0f;
    const bool by4 = NPL % 4 == 0 && N % 4 == 0;
    for (int k = 0; k < ntiles; ++k) {
        const int st = k & 1;
        if (k + 1 < ntiles) load(k + 1, st ^ 1);
        copy_commit();
        copy_wait<1>();
        __syncthreads();
        float* __restrict__ xs = tiles + (size_t)st * stage_floats;
        float* __restrict__ ds = xs + TT * CH;
        float* __restrict__ zs = ds + TT * CH;
        const float* __restrict__ bs = zs + TT * CH;
        const float* __restrict__ cs = bs + TT * N;
        const int t_begin = seg0 + k * TT;
        const int valid = min(TT, seg0 + count - t_begin);
        // (A) step sizes and gates, once a channel
        // (a thread meets the same channel every time: the block's threads are a multiple of CH)
        for (int i = threadIdx.x; i < valid * CH; i += THREADS) {
            if (!mine_live) break;
            ds[i] = softplus_t<FAST>(ds[i] + mine_bias);
            if (!FOLD) zs[i] = silu_t<FAST>(zs[i]);
        }
        __syncthreads();
        // (B) the recurrence: per row NPL independent multiply-adds on S
#pragma unroll 2
        for (int t = 0; t < valid; ++t) {
            const float dt = ds[t * CH + lc];
            const float xt = xs[t * CH + lc];
            const float dx = dt * xt;
            float Bt[NPL], Ct[NPL];
            if (by4) {
#pragma unroll
                for (int i = 0; i < NPL; i += 4) {
                    float4 b4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), c4 = b4;
                    if (n0 + i < N) {
                        b4 = *reinterpret_cast<const float4*>(bs + t * N + n0 + i);
                        if (!FOLD) c4 = *reinterpret_cast<const float4*>(cs + t * N + n0 + i);
                    }
                    Bt[i] = b4.x; Bt[(i + 1) % NPL] = b4.y; Bt[(i + 2) % NPL] = b4.z; Bt[(i + 3) % NPL] = b4.w;
                    Ct[i] = c4.x; Ct[(i + 1) % NPL] = c4.y; Ct[(i + 2) % NPL] = c4.z; Ct[(i + 3) % NPL] = c4.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < NPL; ++i) {
                    Bt[i] = n0 + i < N ? bs[t * N + n0 + i] : 0.0f;
                    Ct[i] = (!FOLD && n0 + i < N) ? cs[t * N + n0 + i] : 0.0f;
                }
            }
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                S[i] = fmaf(decay2(dt * a2[i]), S[i], dx * Bt[i]);
                if (!FOLD) acc = fmaf(S[i], Ct[i], acc);
            }
            if (FOLD) {
                sum_dt += dt;
            } else {
                for (int o = plan.lpc >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (sub == 0) zs[t * CH + lc] = fmaf(d_skip, xt, acc) * zs[t * CH + lc];
            }
        }
        __syncthreads();
        // (C) the tile's results
        if (!FOLD) {
            for (int i = threadIdx.x; i < valid * CH; i += THREADS) {
                const int t = i >> plan.ch_shift, l = i & (CH - 1);
                if (c0 + l < channels) rfx::st<TO>(out, (size_t)(row0 + t_begin + t) * channels + c0 + l, zs[i]);
            }
            __syncthreads();
        }
    }
    copy_wait<0>();
    if (!live) return;
    if (FOLD) {
#pragma unroll
        for (int i = 0; i < NPL; ++i)
            if (n0 + i < N) seg_local[seg_cell * N + n0 + i] = S[i];
        if (sub == 0) seg_dt[seg_cell] = sum_dt;
    } else if (g == G - 1) {
#pragma unroll
        for (int i = 0; i < NPL; ++i)
            if (n0 + i < N) st_c[n0 + i] = S[i];
    }
}

// step (2): a thread a (sequence, channel, state) carries S through the segments
__global__ void __launch_bounds__(256)
mamba_scan_carry_kernel(const float* __restrict__ A, const float* __restrict__ state, size_t slot_stride,
                        size_t state_off, const int* __restrict__ seq_slot, const float* __restrict__ seg_local,
                        const float* __restrict__ seg_dt, float* __restrict__ seg_begin, int channels, int N,
                        int G) {
    pdl_launch_dependents();
    const int s = blockIdx.x;
    const size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
    const size_t per = (size_t)channels * N;
    if (e >= per) return;
    const int c = (int)(e / N);
    const float a2 = A[e] * LOG2E;
    pdl_wait();
    float S = state[(size_t)seq_slot[s] * slot_stride + state_off + e];
    // eight segments' folds and step-size sums are fetched before their chain runs: the
    // chain then waits for one round of loads in eight steps, not for one a step
    for (int g0 = 0; g0 < G; g0 += 8) {
        float local[8], sum_dt[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const size_t cell = (size_t)s * G + g0 + j;
            const bool on = g0 + j < G - 1;
            local[j] = on ? seg_local[cell * per + e] : 0.0f;
            sum_dt[j] = on ? seg_dt[cell * channels + c] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (g0 + j < G) {
                seg_begin[((size_t)s * G + g0 + j) * per + e] = S;
                S = fmaf(decay2(a2 * sum_dt[j]), S, local[j]);
            }
        }
    }
}

}  // namespace

// how a step of R rows in S sequences is laid out; G = 0: the row-by-row form
static ScanPlan scan_plan(int S, int R, int channels, int N) {
    ScanPlan p{};
    if (R < 4 * S) return p;
    p.lpc = 1;
    while (p.lpc < 32 && p.lpc * 16 < N) p.lpc <<= 1;
    for (int v = p.lpc; v > 1; v >>= 1) ++p.lp_shift;
    for (int v = THREADS / p.lpc; v > 1; v >>= 1) ++p.ch_shift;
    const int CH = THREADS / p.lpc;
    p.TT = 16;
    while (p.TT > 4 && (size_t)2 * p.TT * (3 * CH + 2 * N) * sizeof(float) > 72 * 1024) p.TT >>= 1;
    // segments: enough for about four warps a scheduler, of 32 rows and more each
    const long long warps = (long long)S * ((channels + CH - 1) / CH) * (THREADS / 32);
    long long G = (rfx::sm_count() * 16 + warps - 1) / warps;
    const long long longest = (R / S) / 32;
    if (G > longest) G = longest;
    if (G > 64) G = 64;
    if (G < 1) G = 1;
    p.G = (int)G;
    return p;
}

// floats of scratch that rfx_mamba_scan wants for this step (0: none)
extern "C" long long rfx_mamba_scan_scratch(int S, int R, int channels, int N) {
    if (S <= 0 || channels <= 0 || N < 1 || N > 512) return 0;
    const ScanPlan p = scan_plan(S, R, channels, N);
    if (p.G <= 1) return 0;
    return (long long)S * p.G * channels * (2LL * N + 1);
}

// x, dtpre: float32 [R][channels].  `bc`: float32 rows of `ld_bc` floats that hold
// B at column `b_off` and C at `c_off` (N each).  `zsrc`: float32 rows of `ld_z`
// floats with z at column `z_off`.  A: [channels][N] (negative).  `state`:
// [slots][slot_stride] floats, this mixer's S at `state_off`.  R rows in all, of S
// sequences: steps of four rows a sequence and more take the tiled form, which
// wants `scratch` (rfx_mamba_scan_scratch floats) when it cuts sequences into segments.
// `w_dt` (may be null; then `dtpre` holds the step sizes before their bias): W_dt
// [channels][rank] of type `w_dt_type`; the rows of `bc` hold the low-rank vector at
// column `low_off`, and dtpre = W_dt . vector is made here (row-by-row form only).
extern "C" int rfx_mamba_scan(const float* x, const float* dtpre, const float* dt_bias, const float* bc,
                              int ld_bc, int b_off, int c_off, const float* zsrc, int ld_z, int z_off,
                              const float* A, const float* Dw, float* state, long long slot_stride,
                              long long state_off, const int* seq_slot, const int* seq_row0, int S, int R,
                              void* out, int out_dt, int channels, int N, float* scratch, const void* w_dt,
                              int w_dt_type, int rank, int low_off, void* stream) {
    if (S <= 0 || channels <= 0) return 0;
    if (N < 1 || N > 512) return RFX_ERR_UNSUPPORTED;
    if (out_dt != RFX_DT_F32 && out_dt != RFX_DT_BF16) return RFX_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const ScanPlan plan = scan_plan(S, R, channels, N);
    StepRank sr{};
    if (w_dt) {
        // the step sizes' last product rides in the row-by-row form only
        if (plan.G >= 1) return RFX_ERR_UNSUPPORTED;
        if ((w_dt_type != RFX_DT_F32 && w_dt_type != RFX_DT_BF16) || rank < 1 || low_off < 0 || low_off + rank > ld_bc)
            return RFX_ERR_BAD_ARG;
        sr.w = w_dt;
        sr.bf16 = w_dt_type == RFX_DT_BF16;
        sr.rank = rank;
        sr.off = low_off;
    } else if (!dtpre) {
        return RFX_ERR_BAD_ARG;
    }
    if (plan.G >= 1) {
        const int lpc = plan.lpc, CH = THREADS / lpc, TT = plan.TT, G = plan.G;
        const int npl = (N + lpc - 1) / lpc;
        const size_t smem = (size_t)2 * TT * (3 * CH + 2 * N) * sizeof(float);
        const dim3 grid(S, (channels + CH - 1) / CH, G);
        if (grid.y > 65535 || smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
        if (G > 1 && !scratch) return RFX_ERR_BAD_ARG;
        const size_t cells = (size_t)S * G * channels;
        float* seg_local = scratch;
        float* seg_begin = scratch ? scratch + cells * N : nullptr;
        float* seg_dt = scratch ? scratch + 2 * cells * N : nullptr;
        auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
        const bool wide = channels % 4 == 0 && N % 4 == 0 && ld_bc % 4 == 0 && b_off % 4 == 0 && c_off % 4 == 0 &&
                          ld_z % 4 == 0 && z_off % 4 == 0 && aligned(x) && aligned(dtpre) && aligned(bc) &&
                          aligned(zsrc);
#define RFX_TILED(TO, P, V, FOLD, FAST)                                                                           \
    do {                                                                                                          \
        if (smem > 48 * 1024)                                                                                     \
            cudaFuncSetAttribute(mamba_scan_tiled_kernel<TO, P, V, FOLD, FAST>,                                   \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                         \
        RFX_LAUNCH((mamba_scan_tiled_kernel<TO, P, V, FOLD, FAST>), grid, THREADS, smem, st, x, dtpre, dt_bias,   \
                   bc, ld_bc, b_off, c_off, zsrc, ld_z, z_off, A, Dw, state, (size_t)slot_stride,                 \
                   (size_t)state_off, seq_slot, seq_row0, (TO*)out, channels, N, plan, seg_local, seg_dt,         \
                   (const float*)seg_begin);                                                                      \
    } while (0)
#define RFX_TILED_N(TO, V, FOLD, FAST)                       \
    do {                                                     \
        if (npl <= 1) RFX_TILED(TO, 1, V, FOLD, FAST);       \
        else if (npl <= 2) RFX_TILED(TO, 2, V, FOLD, FAST);  \
        else if (npl <= 4) RFX_TILED(TO, 4, V, FOLD, FAST);  \
        else if (npl <= 8) RFX_TILED(TO, 8, V, FOLD, FAST);  \
        else RFX_TILED(TO, 16, V, FOLD, FAST);               \
    } while (0)
        const bool fast = out_dt == RFX_DT_BF16;
        if (G > 1) {
            // the fold writes no rows: one output type serves
            if (wide && fast) RFX_TILED_N(float, 4, true, true);
            else if (wide) RFX_TILED_N(float, 4, true, false);
            else if (fast) RFX_TILED_N(float, 1, true, true);
            else RFX_TILED_N(float, 1, true, false);
            const size_t per = (size_t)channels * N;
            RFX_LAUNCH(mamba_scan_carry_kernel, dim3(S, (unsigned)((per + 255) / 256)), 256, 0, st, A,
                       (const float*)state, (size_t)slot_stride, (size_t)state_off, seq_slot,
                       (const float*)seg_local, (const float*)seg_dt, seg_begin, channels, N, G);
        }
        if (out_dt == RFX_DT_F32) {
            if (wide) RFX_TILED_N(float, 4, false, false);
            else RFX_TILED_N(float, 1, false, false);
        } else {
            if (wide) RFX_TILED_N(__nv_bfloat16, 4, false, true);
            else RFX_TILED_N(__nv_bfloat16, 1, false, true);
        }
#undef RFX_TILED_N
#undef RFX_TILED
        return 0;
    }
    // four states a lane where the channel's lanes reach; more beyond 128 states
    int lpc = 1;
    while (lpc < 32 && lpc * 4 < N) lpc <<= 1;
    const int npl = (N + lpc - 1) / lpc;
    const dim3 grid(S, (channels + THREADS / lpc - 1) / (THREADS / lpc));
    if (grid.y > 65535) return RFX_ERR_UNSUPPORTED;
#define RFX_SCAN(TO, P)                                                                                       \
    RFX_LAUNCH((mamba_scan_kernel<TO, P>), grid, THREADS, 0, st, x, dtpre, dt_bias, bc, ld_bc, b_off, c_off, \
               zsrc, ld_z, z_off, A, Dw, state, (size_t)slot_stride, (size_t)state_off, seq_slot, seq_row0,  \
               (TO*)out, channels, N, lpc, sr)
#define RFX_SCAN_N(TO)                       \
    do {                                     \
        if (npl <= 1) RFX_SCAN(TO, 1);       \
        else if (npl <= 2) RFX_SCAN(TO, 2);  \
        else if (npl <= 4) RFX_SCAN(TO, 4);  \
        else if (npl <= 8) RFX_SCAN(TO, 8);  \
        else RFX_SCAN(TO, 16);               \
    } while (0)
    if (out_dt == RFX_DT_F32) RFX_SCAN_N(float);
    else RFX_SCAN_N(__nv_bfloat16);
#undef RFX_SCAN_N
#undef RFX_SCAN
    return 0;
}
