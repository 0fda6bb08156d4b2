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
// A block owns (sequence, head, slice of CW value channels) and walks the
// sequence's rows in order with its columns of S in shared memory.  Thread
// (g, j) takes the key channels i = g, g + KG, ... of column j; the KG partial
// sums of u^T S and of S^T r meet in shared memory in index order.
#include "common.cuh"

namespace {

using namespace rfx;

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

}  // namespace

extern "C" int rfx_delta_rule(const float* proj, int ld, int r_off, int k_off, int v_off, int a_off,
                              const float* wpre, const float* w_bias, const float* a_bias, float rate,
                              float unit_eps, float* state, long long state_stride, long long state_off,
                              const int* seq_slot, const int* seq_row0, int n_seq, void* out, int out_dt,
                              int heads, int d, void* stream) {
    if (n_seq <= 0) return 0;
    if (heads <= 0 || d <= 0) return RFX_ERR_BAD_ARG;
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
