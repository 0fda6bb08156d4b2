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

}  // namespace

// x, dtpre: float32 [R][channels].  `bc`: float32 rows of `ld_bc` floats that hold
// B at column `b_off` and C at `c_off` (N each).  `zsrc`: float32 rows of `ld_z`
// floats with z at column `z_off`.  A: [channels][N] (negative).  `state`:
// [slots][slot_stride] floats, this mixer's S at `state_off`.
extern "C" int rfx_mamba_scan(const float* x, const float* dtpre, const float* dt_bias, const float* bc,
                              int ld_bc, int b_off, int c_off, const float* zsrc, int ld_z, int z_off,
                              const float* A, const float* Dw, float* state, long long slot_stride,
                              long long state_off, const int* seq_slot, const int* seq_row0, int S, void* out,
                              int out_dt, int channels, int N, void* stream) {
    if (S <= 0 || channels <= 0) return 0;
    if (N < 1 || N > 512) return RFX_ERR_UNSUPPORTED;
    // four states a lane where the channel's lanes reach; more beyond 128 states
    int lpc = 1;
    while (lpc < 32 && lpc * 4 < N) lpc <<= 1;
    const int npl = (N + lpc - 1) / lpc;
    const dim3 grid(S, (channels + THREADS / lpc - 1) / (THREADS / lpc));
    if (grid.y > 65535) return RFX_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
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
