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
// Prompts take the tiled form: a block walks its sequence in tiles of TT rows.
// The tile's operands (its channels' x, dt and z, the rows' B and C) arrive in
// shared memory by asynchronous copies while the tile before is computed, so a
// step of the recurrence waits for no load.  Per tile: (A) every thread turns
// some of the tile's dt into softplus(dt + bias) and z into silu(z), each once a
// channel and not once a lane; (B) the recurrence, four rows an iteration so
// that the exponentials and the lanes' shuffles of four rows overlap and only
// the multiply-add on S is a chain; (C) the tile's results leave in row order.
// Both forms do the same 32-bit arithmetic in the same order on S.
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int THREADS = 128;

__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

template <typename TO, int NPL>
__global__ void __launch_bounds__(THREADS)
mamba_scan_kernel(const float* __restrict__ x, const float* __restrict__ dtpre, const float* __restrict__ dt_bias,
                  const float* __restrict__ bc, int ld_bc, int b_off, int c_off,
                  const float* __restrict__ zsrc, int ld_z, int z_off, const float* __restrict__ A,
                  const float* __restrict__ Dw, float* __restrict__ state, size_t slot_stride, size_t state_off,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_row0, TO* __restrict__ out,
                  int channels, int N, int lpc) {
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
        a[i] = n < N ? A[(size_t)cc * N + n] : 0.0f;
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
        dv = dtpre[r * channels + cc];
        zv = zsrc[r * ld_z + z_off + cc];
        const float* brow = bc + r * ld_bc;
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
            S[i] = fmaf(expf(dt * a[i]), S[i], dx * Bt[i]);
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


// ---------------------------------------------------------------- tiled form
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

// V floats a copy: 4 where every address involved is a multiple of 16 bytes, else 1.
template <typename TO, int NPL, int V>
__global__ void __launch_bounds__(THREADS)
mamba_scan_tiled_kernel(const float* __restrict__ x, const float* __restrict__ dtpre,
                        const float* __restrict__ dt_bias, const float* __restrict__ bc, int ld_bc, int b_off,
                        int c_off, const float* __restrict__ zsrc, int ld_z, int z_off,
                        const float* __restrict__ A, const float* __restrict__ Dw, float* __restrict__ state,
                        size_t slot_stride, size_t state_off, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_row0, TO* __restrict__ out, int channels, int N, int lpc,
                        int TT) {
    extern __shared__ float4 tiles4[];
    float* tiles = reinterpret_cast<float*>(tiles4);
    pdl_launch_dependents();
    const int CH = THREADS / lpc;                            // channels of a block
    const int stage_floats = TT * (3 * CH + 2 * N);
    const int s = blockIdx.x;
    const int c0 = blockIdx.y * CH;
    const int lc = threadIdx.x / lpc, sub = threadIdx.x % lpc;
    const int c = c0 + lc;
    const bool live = c < channels;
    const int cc = live ? c : channels - 1;
    float a[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int n = sub + i * lpc;
        a[i] = n < N ? A[(size_t)cc * N + n] : 0.0f;
    }
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
    const int ntiles = (rows + TT - 1) / TT;
    // a tile's operands into stage `g`; rows past the sequence's end and channels past
    // the last one are zeros (a zero step leaves S as it is)
    auto load = [&](int k, int g) {
        float* xs = tiles + (size_t)g * stage_floats;
        float* ds = xs + TT * CH;
        float* zs = ds + TT * CH;
        float* bs = zs + TT * CH;
        float* cs = bs + TT * N;
        const int t_begin = k * TT;
        const int valid = min(TT, rows - t_begin);
        const int padded = min(TT, (valid + 3) & ~3);
        for (int i = threadIdx.x * V; i < padded * CH; i += THREADS * V) {
            const int t = i / CH, l = i % CH;
            const size_t r = (size_t)(row0 + t_begin + t);
            if (t < valid && c0 + l < channels) {
                if (V == 4) {
                    copy_async16(xs + i, x + r * channels + c0 + l);
                    copy_async16(ds + i, dtpre + r * channels + c0 + l);
                    copy_async16(zs + i, zsrc + r * ld_z + z_off + c0 + l);
                } else {
                    copy_async4(xs + i, x + r * channels + c0 + l);
                    copy_async4(ds + i, dtpre + r * channels + c0 + l);
                    copy_async4(zs + i, zsrc + r * ld_z + z_off + c0 + l);
                }
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) xs[i + v] = ds[i + v] = zs[i + v] = 0.0f;
            }
        }
        for (int i = threadIdx.x * V; i < padded * N; i += THREADS * V) {
            const int t = i / N, n = i % N;
            const float* brow = bc + (size_t)(row0 + t_begin + t) * ld_bc;
            if (t < valid) {
                if (V == 4) {
                    copy_async16(bs + i, brow + b_off + n);
                    copy_async16(cs + i, brow + c_off + n);
                } else {
                    copy_async4(bs + i, brow + b_off + n);
                    copy_async4(cs + i, brow + c_off + n);
                }
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) bs[i + v] = cs[i + v] = 0.0f;
            }
        }
    };
    if (ntiles > 0) load(0, 0);
    copy_commit();
    for (int k = 0; k < ntiles; ++k) {
        const int g = k & 1;
        if (k + 1 < ntiles) load(k + 1, g ^ 1);
        copy_commit();
        copy_wait<1>();
        __syncthreads();
        float* xs = tiles + (size_t)g * stage_floats;
        float* ds = xs + TT * CH;
        float* zs = ds + TT * CH;
        const float* bs = zs + TT * CH;
        const float* cs = bs + TT * N;
        const int t_begin = k * TT;
        const int valid = min(TT, rows - t_begin);
        const int padded = min(TT, (valid + 3) & ~3);
        // (A) step sizes and gates, once a channel
        for (int i = threadIdx.x; i < padded * CH; i += THREADS) {
            const int t = i / CH, l = i % CH;
            const int ch = min(c0 + l, channels - 1);
            const float zt = zs[i];
            ds[i] = t < valid ? softplus_f(ds[i] + (dt_bias ? dt_bias[ch] : 0.0f)) : 0.0f;
            zs[i] = zt / (1.0f + expf(-zt));
        }
        __syncthreads();
        // (B) the recurrence, four rows an iteration
        for (int t0 = 0; t0 < padded; t0 += 4) {
            float y[4], xt[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int t = t0 + j;
                const float dt = ds[t * CH + lc];
                xt[j] = xs[t * CH + lc];
                const float dx = dt * xt[j];
                float acc = 0.0f;
#pragma unroll
                for (int i = 0; i < NPL; ++i) {
                    const int n = sub + i * lpc;
                    const float Bt = n < N ? bs[t * N + n] : 0.0f;
                    const float Ct = n < N ? cs[t * N + n] : 0.0f;
                    S[i] = fmaf(expf(dt * a[i]), S[i], dx * Bt);
                    acc = fmaf(S[i], Ct, acc);
                }
                y[j] = acc;
            }
            for (int o = lpc >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) y[j] += __shfl_xor_sync(0xffffffffu, y[j], o);
            }
            if (sub == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = (t0 + j) * CH + lc;
                    zs[i] = fmaf(d_skip, xt[j], y[j]) * zs[i];
                }
            }
        }
        __syncthreads();
        // (C) the tile's results
        for (int i = threadIdx.x; i < valid * CH; i += THREADS) {
            const int t = i / CH, l = i % CH;
            if (c0 + l < channels) rfx::st<TO>(out, (size_t)(row0 + t_begin + t) * channels + c0 + l, zs[i]);
        }
        __syncthreads();
    }
    copy_wait<0>();
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int n = sub + i * lpc;
            if (n < N) st_c[n] = S[i];
        }
    }
}

}  // namespace

// x, dtpre: float32 [R][channels].  `bc`: float32 rows of `ld_bc` floats that hold
// B at column `b_off` and C at `c_off` (N each).  `zsrc`: float32 rows of `ld_z`
// floats with z at column `z_off`.  A: [channels][N] (negative).  `state`:
// [slots][slot_stride] floats, this mixer's S at `state_off`.  R rows in all, of S
// sequences: steps of four rows a sequence and more take the tiled form.
extern "C" int rfx_mamba_scan(const float* x, const float* dtpre, const float* dt_bias, const float* bc,
                              int ld_bc, int b_off, int c_off, const float* zsrc, int ld_z, int z_off,
                              const float* A, const float* Dw, float* state, long long slot_stride,
                              long long state_off, const int* seq_slot, const int* seq_row0, int S, int R,
                              void* out, int out_dt, int channels, int N, void* stream) {
    if (S <= 0 || channels <= 0) return 0;
    if (N < 1 || N > 512) return RFX_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (R >= 4 * S) {
        // prompts: the tiled form, two states a lane where the channel's lanes reach
        int lpc = 1;
        while (lpc < 32 && lpc * 2 < N) lpc <<= 1;
        const int npl = (N + lpc - 1) / lpc;
        const int CH = THREADS / lpc;
        int TT = 32;
        while (TT > 4 && (size_t)2 * TT * (3 * CH + 2 * N) * sizeof(float) > 160 * 1024) TT >>= 1;
        const size_t smem = (size_t)2 * TT * (3 * CH + 2 * N) * sizeof(float);
        const dim3 grid(S, (channels + CH - 1) / CH);
        if (grid.y > 65535 || smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
        auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
        const bool wide = CH % 4 == 0 && channels % 4 == 0 && N % 4 == 0 && ld_bc % 4 == 0 && b_off % 4 == 0 &&
                          c_off % 4 == 0 && ld_z % 4 == 0 && z_off % 4 == 0 && aligned(x) && aligned(dtpre) &&
                          aligned(bc) && aligned(zsrc);
#define RFX_TILED(TO, P, V)                                                                                    \
    do {                                                                                                       \
        if (smem > 48 * 1024)                                                                                  \
            cudaFuncSetAttribute(mamba_scan_tiled_kernel<TO, P, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                   \
        RFX_LAUNCH((mamba_scan_tiled_kernel<TO, P, V>), grid, THREADS, smem, st, x, dtpre, dt_bias, bc, ld_bc,  \
                   b_off, c_off, zsrc, ld_z, z_off, A, Dw, state, (size_t)slot_stride, (size_t)state_off,      \
                   seq_slot, seq_row0, (TO*)out, channels, N, lpc, TT);                                        \
    } while (0)
#define RFX_TILED_N(TO, V)                       \
    do {                                         \
        if (npl <= 1) RFX_TILED(TO, 1, V);       \
        else if (npl <= 2) RFX_TILED(TO, 2, V);  \
        else if (npl <= 4) RFX_TILED(TO, 4, V);  \
        else if (npl <= 8) RFX_TILED(TO, 8, V);  \
        else RFX_TILED(TO, 16, V);               \
    } while (0)
        if (out_dt == RFX_DT_F32) {
            if (wide) RFX_TILED_N(float, 4);
            else RFX_TILED_N(float, 1);
        } else if (out_dt == RFX_DT_BF16) {
            if (wide) RFX_TILED_N(__nv_bfloat16, 4);
            else RFX_TILED_N(__nv_bfloat16, 1);
        } else {
            return RFX_ERR_BAD_ARG;
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
               (TO*)out, channels, N, lpc)
#define RFX_SCAN_N(TO)                       \
    do {                                     \
        if (npl <= 1) RFX_SCAN(TO, 1);       \
        else if (npl <= 2) RFX_SCAN(TO, 2);  \
        else if (npl <= 4) RFX_SCAN(TO, 4);  \
        else if (npl <= 8) RFX_SCAN(TO, 8);  \
        else RFX_SCAN(TO, 16);               \
    } while (0)
    if (out_dt == RFX_DT_F32) RFX_SCAN_N(float);
    else if (out_dt == RFX_DT_BF16) RFX_SCAN_N(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_SCAN_N
#undef RFX_SCAN
    return 0;
}
