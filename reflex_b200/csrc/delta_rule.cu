// The generalized delta rule: a matrix memory per head with a decay and a removal
// rate per key channel.
//
// Per head, with d key channels and d value channels, and for every row
//     w = exp(-rate * sigmoid(w_pre + w_bias))        decay per key channel
//     a = sigmoid(a_pre + a_bias)                     removal rate per key channel
//     u = k / sqrt(sum(k^2) + unit_eps)               the unit key
//     S <- diag(w) S - (a * u) (u^T S) + k v^T        (both terms read the old S)
//     o = S^T r
// `proj` holds float32 rows with r, k, v and a_pre at their column offsets
// (heads * d each); `wpre` float32 rows [heads * d].  The running state is
// `state[slot * stride + off ...]`, [heads][d][d] float32 (key channel, value
// channel), carried from step to step.  `rate` and `unit_eps` are the caller's
// constants.  Everything is 32-bit.
//
// Two forms.  The one below the general one takes head sizes that are a multiple
// of four (see there).  The general one:
// a block owns (sequence, head, slice of CW value channels) and walks the
// sequence's rows in order with its columns of S in shared memory.  Thread
// (g, j) takes the key channels i = g, g + KG, ... of column j; the KG partial
// sums of u^T S and of S^T r meet in shared memory in index order.
#include "common.cuh"

namespace {

using namespace rfx;

// fewest warps a block of the warp-walking form keeps when its columns are cut further to fill
// the SMs (REFLEX_B200_SCAN_MIN_WARPS, a tuning aid read once)
inline int scan_min_warps() {
    static int v = 0;
    if (!v) {
        const char* e = getenv("REFLEX_B200_SCAN_MIN_WARPS");
        v = e ? atoi(e) : 16;
        if (v < 1 || v > 16) v = 16;
    }
    return v;
}

__device__ __forceinline__ float sigmoid_f(float t) { return 1.0f / (1.0f + expf(-t)); }

template <typename TO>
__global__ void __launch_bounds__(512)
delta_rule_kernel(const float* __restrict__ proj, int ld, int r_off, int k_off, int v_off, int a_off,
                  const float* __restrict__ wpre, const float* __restrict__ w_bias, const float* __restrict__ a_bias,
                  float rate, float unit_eps, float* __restrict__ state, long long state_stride, long long state_off,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_row0, TO* __restrict__ out,
                  int heads, int d, int CW, int KG) {
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                       // [d][CW]
    float* ws = S + (size_t)d * CW;      // [d] decay
    float* au = ws + d;                  // [d] a * u
    float* us = au + d;                  // [d] u
    float* ks = us + d;                  // [d] k
    float* rs = ks + d;                  // [d] r
    float* part = rs + d;                // [KG][CW]
    float* sa = part + (size_t)KG * CW;  // [CW] u^T S
    __shared__ float scratch[32];
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CW;
    const int tid = threadIdx.x, j = tid % CW, g = tid / CW;
    const int row0 = seq_row0[seq], row1 = seq_row0[seq + 1];
    const int hd = heads * d;
    float* Sg = state + (size_t)seq_slot[seq] * state_stride + state_off + (size_t)h * d * d;
    for (int i = tid; i < d * CW; i += blockDim.x) {
        const int n = i / CW, c = i - n * CW;
        S[i] = Sg[(size_t)n * d + c0 + c];
    }
    for (int r = row0; r < row1; ++r) {
        const float* pr = proj + (size_t)r * ld + h * d;
        float kk = 0.0f;
        for (int i = tid; i < d; i += blockDim.x) {
            const float kv = pr[k_off + i];
            kk = fmaf(kv, kv, kk);
        }
        // block_sum's barriers also separate the row before from this row's vectors
        const float inv = 1.0f / sqrtf(block_sum(kk, scratch) + unit_eps);
        for (int i = tid; i < d; i += blockDim.x) {
            const float kv = pr[k_off + i];
            const float u = kv * inv;
            ks[i] = kv;
            us[i] = u;
            au[i] = sigmoid_f(pr[a_off + i] + a_bias[h * d + i]) * u;
            ws[i] = expf(-rate * sigmoid_f(wpre[(size_t)r * hd + h * d + i] + w_bias[h * d + i]));
            rs[i] = pr[r_off + i];
        }
        __syncthreads();
        float acc = 0.0f;
        for (int i = g; i < d; i += KG) acc = fmaf(us[i], S[i * CW + j], acc);
        part[g * CW + j] = acc;
        __syncthreads();
        if (g == 0) {
            float t = 0.0f;
            for (int q = 0; q < KG; ++q) t += part[q * CW + j];
            sa[j] = t;
        }
        __syncthreads();
        const float saj = sa[j], vj = pr[v_off + c0 + j];
        acc = 0.0f;
        for (int i = g; i < d; i += KG) {
            const float s = fmaf(ks[i], vj, fmaf(ws[i], S[i * CW + j], -au[i] * saj));
            S[i * CW + j] = s;
            acc = fmaf(s, rs[i], acc);
        }
        part[g * CW + j] = acc;
        __syncthreads();
        if (g == 0) {
            float t = 0.0f;
            for (int q = 0; q < KG; ++q) t += part[q * CW + j];
            st<TO>(out, (size_t)r * hd + h * d + c0 + j, t);
        }
    }
    __syncthreads();
    for (int i = tid; i < d * CW; i += blockDim.x) {
        const int n = i / CW, c = i - n * CW;
        Sg[(size_t)n * d + c0 + c] = S[i];
    }
}


// ---- the form for head sizes that are a multiple of four, up to 256 ------------
// A block owns (sequence, head, some of the value columns) and walks the rows in
// tiles of TT: all its threads first stage a tile (k, a, w, r and v of its rows into
// shared memory, 16 bytes a load, then a warp a row: the unit key's norm by the lanes'
// butterfly, u and a * u), then each warp walks the tile's rows on its own four
// columns (four, two or one) with no further barrier: KG lanes (8, 16 or 32) share a
// column, lane (g, c) holds its key channels 4 (g + KG m) .. + 3 in registers (NC groups
// of four, read from the tile 16 bytes at a time), the KG partial sums of u^T S and of
// S^T r meet by shuffles.  The state
// lies [heads][value column][key channel].  Which block and warp walks a column
// changes nothing of its arithmetic.
template <int NC, int KG, typename TO>
__global__ void __launch_bounds__(512)
delta_rule_warp_kernel(const float* __restrict__ proj, int ld, int r_off, int k_off, int v_off, int a_off,
                       const float* __restrict__ wpre, const float* __restrict__ w_bias,
                       const float* __restrict__ a_bias, float rate, float unit_eps, float* __restrict__ state,
                       long long state_stride, long long state_off, const int* __restrict__ seq_slot,
                       const int* __restrict__ seq_row0, TO* __restrict__ out, int heads, int d, int cols, int TT) {
    extern __shared__ __align__(16) float sm[];  // [TT][6][d]: k, u, a * u, w, r, v
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y, c_first = blockIdx.z * cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    constexpr int CW = 32 / KG;  // columns a warp walks; KG lanes share a column
    const int g = lane / CW, col = c_first + warp * CW + (lane % CW);
    const int row0 = seq_row0[seq], row1 = seq_row0[seq + 1];
    const int hd = heads * d, d4 = d / 4;
    float* Sg = state + (size_t)seq_slot[seq] * state_stride + state_off + ((size_t)h * d + col) * d;
    float S[NC][4];
#pragma unroll
    for (int m = 0; m < NC; ++m)
#pragma unroll
        for (int q = 0; q < 4; ++q) S[m][q] = g + KG * m < d4 ? Sg[4 * (g + KG * m) + q] : 0.0f;
    const float4* ab4 = reinterpret_cast<const float4*>(a_bias + h * d);
    const float4* wb4 = reinterpret_cast<const float4*>(w_bias + h * d);
    for (int t0 = row0; t0 < row1; t0 += TT) {
        const int nt = min(TT, row1 - t0);
        __syncthreads();  // the tile before has been walked by every warp
        // four neighbouring elements by whichever thread comes to them: all their loads
        // first, then the arithmetic, so that many rows' loads are in flight together
#pragma unroll 2
        for (int e = threadIdx.x; e < nt * d4; e += blockDim.x) {
            const int t = e / d4, c = e - t * d4;
            const float* pr = proj + (size_t)(t0 + t) * ld + h * d;
            const float4 kv = reinterpret_cast<const float4*>(pr + k_off)[c];
            const float4 ap = reinterpret_cast<const float4*>(pr + a_off)[c];
            const float4 rv = reinterpret_cast<const float4*>(pr + r_off)[c];
            const float4 vv = reinterpret_cast<const float4*>(pr + v_off)[c];
            const float4 wv = reinterpret_cast<const float4*>(wpre + (size_t)(t0 + t) * hd + h * d)[c];
            const float4 ab = ab4[c], wb = wb4[c];
            float4* tile = reinterpret_cast<float4*>(sm + (size_t)t * 6 * d);
            tile[c] = kv;
            tile[2 * d4 + c] = make_float4(sigmoid_f(ap.x + ab.x), sigmoid_f(ap.y + ab.y), sigmoid_f(ap.z + ab.z),
                                           sigmoid_f(ap.w + ab.w));  // a; times u below
            tile[3 * d4 + c] = make_float4(expf(-rate * sigmoid_f(wv.x + wb.x)), expf(-rate * sigmoid_f(wv.y + wb.y)),
                                           expf(-rate * sigmoid_f(wv.z + wb.z)), expf(-rate * sigmoid_f(wv.w + wb.w)));
            tile[4 * d4 + c] = rv;
            tile[5 * d4 + c] = vv;
        }
        __syncthreads();
        // a warp a row: the unit key by the lanes' butterfly
        for (int t = warp; t < nt; t += nwarps) {
            float* tile = sm + (size_t)t * 6 * d;
            float kk = 0.0f;
            for (int i = lane; i < d; i += 32) kk = fmaf(tile[i], tile[i], kk);
            const float inv = 1.0f / sqrtf(warp_sum(kk) + unit_eps);
            for (int i = lane; i < d; i += 32) {
                const float u = tile[i] * inv;
                tile[d + i] = u;
                tile[2 * d + i] *= u;
            }
        }
        __syncthreads();
        // four rows at a time: u^T S must meet before the state's step (one chain of shuffles a
        // row), the rows' partial sums of S^T r meet together afterwards (their chains side by side)
        for (int t = 0; t < nt; t += 4) {
            float ov[4];
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) {
                ov[u4] = 0.0f;
                if (t + u4 < nt) {
                    const float4* tile = reinterpret_cast<const float4*>(sm + (size_t)(t + u4) * 6 * d);
                    float acc = 0.0f, acc1 = 0.0f;
#pragma unroll
                    for (int m = 0; m < NC; ++m) {
                        const int c = g + KG * m;
                        if (c < d4) {
                            const float4 u = tile[d4 + c];
                            acc = fmaf(u.x, S[m][0], fmaf(u.y, S[m][1], acc));
                            acc1 = fmaf(u.z, S[m][2], fmaf(u.w, S[m][3], acc1));
                        }
                    }
                    acc += acc1;
#pragma unroll
                    for (int off = CW; off < 32; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                    const float vj = reinterpret_cast<const float*>(tile)[5 * d + col];
                    float o = 0.0f, o1 = 0.0f;
#pragma unroll
                    for (int m = 0; m < NC; ++m) {
                        const int c = g + KG * m;
                        if (c < d4) {
                            const float4 k = tile[c], au = tile[2 * d4 + c], w = tile[3 * d4 + c], r = tile[4 * d4 + c];
                            S[m][0] = fmaf(k.x, vj, fmaf(w.x, S[m][0], -au.x * acc));
                            S[m][1] = fmaf(k.y, vj, fmaf(w.y, S[m][1], -au.y * acc));
                            S[m][2] = fmaf(k.z, vj, fmaf(w.z, S[m][2], -au.z * acc));
                            S[m][3] = fmaf(k.w, vj, fmaf(w.w, S[m][3], -au.w * acc));
                            o = fmaf(S[m][0], r.x, fmaf(S[m][1], r.y, o));
                            o1 = fmaf(S[m][2], r.z, fmaf(S[m][3], r.w, o1));
                        }
                    }
                    ov[u4] = o + o1;
                }
            }
#pragma unroll
            for (int off = CW; off < 32; off <<= 1)
#pragma unroll
                for (int u4 = 0; u4 < 4; ++u4) ov[u4] += __shfl_xor_sync(0xffffffffu, ov[u4], off);
            if (g == 0) {
#pragma unroll
                for (int u4 = 0; u4 < 4; ++u4)
                    if (t + u4 < nt) st<TO>(out, (size_t)(t0 + t + u4) * hd + h * d + col, ov[u4]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < NC; ++m)
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (g + KG * m < d4) Sg[4 * (g + KG * m) + q] = S[m][q];
}

template <int NC, int KG, typename TO>
int launch_warp(const float* proj, int ld, int r_off, int k_off, int v_off, int a_off, const float* wpre,
                const float* w_bias, const float* a_bias, float rate, float unit_eps, float* state,
                long long state_stride, long long state_off, const int* seq_slot, const int* seq_row0, int n_seq,
                void* out, int heads, int d, cudaStream_t s) {
    // value columns a block owns (four a warp): fewer while the blocks do not fill the SMs
    constexpr int CW = 32 / KG;  // columns a warp
    int cols = d;
    while (cols > 16 * CW && cols % (2 * CW) == 0) cols /= 2;  // at most 16 warps a block
    if (cols > 16 * CW || d % cols) return RFX_ERR_UNSUPPORTED;
    while (cols % (2 * CW) == 0 && cols > scan_min_warps() * CW && (long long)n_seq * heads * (d / cols) < sm_count())
        cols /= 2;
    int TT = (48 * 1024) / (6 * d * (int)sizeof(float));
    if (TT > 32) TT = 32;
    if (TT < 1) TT = 1;
    const size_t smem = (size_t)TT * 6 * d * sizeof(float);
    auto kernel = delta_rule_warp_kernel<NC, KG, TO>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_seq, heads, d / cols);
    RFX_LAUNCH(kernel, grid, (cols / CW) * 32, smem, s, proj, ld, r_off, k_off, v_off, a_off, wpre, w_bias, a_bias,
               rate, unit_eps, state, state_stride, state_off, seq_slot, seq_row0, (TO*)out, heads, d, cols, TT);
    return 0;
}

}  // namespace

extern "C" int rfx_delta_rule(const float* proj, int ld, int r_off, int k_off, int v_off, int a_off,
                              const float* wpre, const float* w_bias, const float* a_bias, float rate,
                              float unit_eps, float* state, long long state_stride, long long state_off,
                              const int* seq_slot, const int* seq_row0, int n_seq, void* out, int out_dt,
                              int heads, int d, void* stream) {
    if (n_seq <= 0) return 0;
    if (heads <= 0 || d <= 0) return RFX_ERR_BAD_ARG;
    const bool aligned = ((ld | r_off | k_off | v_off | a_off) & 3) == 0 &&
                         ((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(wpre) |
                           reinterpret_cast<uintptr_t>(w_bias) | reinterpret_cast<uintptr_t>(a_bias)) & 15) == 0;
    if (d % 4 == 0 && d <= 256 && out_dt == RFX_DT_F32 && aligned) {
#define RFX_WARP(N, G)                                                                                        \
    st = launch_warp<N, G, float>(proj, ld, r_off, k_off, v_off, a_off, wpre, w_bias, a_bias, rate, unit_eps, \
                                  state, state_stride, state_off, seq_slot, seq_row0, n_seq, out, heads, d,   \
                                  (cudaStream_t)stream)
        int st;  // a head size whose columns do not divide among the warps goes to the general form
        // as many lanes a column as it has groups of four key channels (8, 16 or 32): a lane's share
        // is one or two groups, and a head gives enough warps to keep the SMs' schedulers busy
        // (measured at 2,048 rows of 32 heads of 64: 1.0 ms with eight lanes a column and two groups
        // a lane, 2.0 ms with two lanes and eight groups)
        if (d <= 32) RFX_WARP(1, 8);
        else if (d <= 64) RFX_WARP(1, 16);
        else if (d <= 128) RFX_WARP(1, 32);
        else RFX_WARP(2, 32);
        if (st != RFX_ERR_UNSUPPORTED) return st;
#undef RFX_WARP
    }
    // the slice of value channels a block owns, fixed by d alone
    int CW = d;
    while (CW > 32 && CW % 2 == 0) CW /= 2;
    if (CW > 512) return RFX_ERR_UNSUPPORTED;
    int KG = 256 / CW;
    if (KG < 1) KG = 1;
    if (KG > d) KG = d;
    const int threads = KG * CW;
    const size_t smem = ((size_t)d * CW + 5 * (size_t)d + (size_t)KG * CW + CW) * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    dim3 grid(n_seq, heads, d / CW);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(TO)                                                                                           \
    do {                                                                                                     \
        if (smem > 48 * 1024) {                                                                              \
            cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<TO>,                                      \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
            if (e != cudaSuccess) return (int)e;                                                             \
        }                                                                                                    \
        RFX_LAUNCH(delta_rule_kernel<TO>, grid, threads, smem, s, proj, ld, r_off, k_off, v_off, a_off, wpre,  \
                   w_bias, a_bias, rate, unit_eps, state, state_stride, state_off, seq_slot, seq_row0,       \
                   (TO*)out, heads, d, CW, KG);                                                              \
    } while (0)
    if (out_dt == RFX_DT_F32) RFX_GO(float);
    else if (out_dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}
