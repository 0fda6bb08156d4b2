// The state-space recurrence with one decay a head (the "state-space duality"
// form of a selective scan).
//
// Per head h with P value channels, N states and the B, C vectors of its group
// g = h / (heads / groups):
//     dt  = softplus(dt_pre[h] + dt_bias[h])                (no clamp)
//     S  <- exp(A[h] dt) S + dt B x^T                        (S is N x P, A[h] < 0)
//     y   = S^T C + D[h] x
//     out = y * silu(z)
// Inputs: `xbc` float32 rows [x: heads * P | B: groups * N | C: groups * N] (after
// their convolution and activation), `proj` float32 rows holding z at column
// `z_off` (heads * P wide) and dt_pre at `dt_off` (heads wide).  The running state
// is `state[slot * stride + off ...]`, [heads][N][P] float32, carried from step to
// step.  Everything is 32-bit.
//
// A block owns (sequence, head, slice of the P channels) and walks the
// sequence's rows in order; its part of S lives in shared memory; thread
// (k, p) takes the states n = k, k + KG, ... of channel p, and the KG partial
// sums of y meet in shared memory in index order, so a row's result does not
// depend on how the work was cut into steps or on what else is in the batch.
#include "common.cuh"

namespace {

using namespace rfx;

__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

template <typename TO>
__global__ void __launch_bounds__(512)
ssd_scan_kernel(const float* __restrict__ xbc, int ldx, const float* __restrict__ proj, int ldp, int z_off, int dt_off,
                const float* __restrict__ dt_bias, const float* __restrict__ A, const float* __restrict__ D,
                float* __restrict__ state, long long state_stride, long long state_off,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_row0, TO* __restrict__ out,
                int heads, int P, int N, int groups, int PW, int KG) {
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                 // [N][PW]
    float* Bs = S + (size_t)N * PW;  // [N]
    float* Cs = Bs + N;            // [N]
    float* xs = Cs + N;            // [PW]
    float* part = xs + PW;         // [KG][PW]
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PW;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int tid = threadIdx.x, p = tid % PW, k = tid / PW;
    const int row0 = seq_row0[seq], row1 = seq_row0[seq + 1];
    float* Sg = state + (size_t)seq_slot[seq] * state_stride + state_off + (size_t)h * N * P;
    for (int i = tid; i < N * PW; i += blockDim.x) {
        const int n = i / PW, c = i - n * PW;
        S[i] = p0 + c < P ? Sg[(size_t)n * P + p0 + c] : 0.0f;
    }
    const float a = A[h], dcoef = D ? D[h] : 0.0f, bias = dt_bias ? dt_bias[h] : 0.0f;
    for (int r = row0; r < row1; ++r) {
        __syncthreads();  // the row before is done with Bs, Cs, xs and part (and S is loaded)
        const float* xr = xbc + (size_t)r * ldx;
        for (int i = tid; i < N; i += blockDim.x) {
            Bs[i] = xr[inner + g * N + i];
            Cs[i] = xr[inner + groups * N + g * N + i];
        }
        for (int i = tid; i < PW; i += blockDim.x) xs[i] = p0 + i < P ? xr[h * P + p0 + i] : 0.0f;
        const float dt = softplus_f(proj[(size_t)r * ldp + dt_off + h] + bias);
        const float decay = expf(a * dt);
        __syncthreads();
        const float dx = dt * xs[p];
        float acc = 0.0f;
        for (int n = k; n < N; n += KG) {
            const float s = fmaf(S[n * PW + p], decay, Bs[n] * dx);
            S[n * PW + p] = s;
            acc = fmaf(s, Cs[n], acc);
        }
        part[k * PW + p] = acc;
        __syncthreads();
        if (k == 0 && p0 + p < P) {
            float y = 0.0f;
            for (int j = 0; j < KG; ++j) y += part[j * PW + p];
            y = fmaf(dcoef, xs[p], y);
            const float z = proj[(size_t)r * ldp + z_off + h * P + p0 + p];
            st<TO>(out, (size_t)r * inner + h * P + p0 + p, y * (z / (1.0f + expf(-z))));
        }
    }
    __syncthreads();
    for (int i = tid; i < N * PW; i += blockDim.x) {
        const int n = i / PW, c = i - n * PW;
        if (p0 + c < P) Sg[(size_t)n * P + p0 + c] = S[i];
    }
}

}  // namespace

extern "C" int rfx_ssd_scan(const float* xbc, int ldx, const float* proj, int ldp, int z_off, int dt_off,
                            const float* dt_bias, const float* A, const float* D, float* state,
                            long long state_stride, long long state_off, const int* seq_slot, const int* seq_row0,
                            int n_seq, void* out, int out_dt, int heads, int P, int N, int groups, void* stream) {
    if (n_seq <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0) return RFX_ERR_BAD_ARG;
    // the slice of channels a block owns, fixed by P alone: how a row's sums are ordered
    // does not depend on what else is in the step
    int PW = P;
    while (PW > 32 && PW % 2 == 0) PW /= 2;
    const int slices = (P + PW - 1) / PW;
    int KG = 256 / PW;
    if (KG < 1) KG = 1;
    if (KG > N) KG = N;
    while ((long long)KG * PW > 512) --KG;
    if (KG < 1) return RFX_ERR_UNSUPPORTED;  // more than 512 channels a slice cannot be
    const int threads = KG * PW;
    const size_t smem = ((size_t)N * PW + 2 * (size_t)N + PW + (size_t)KG * PW) * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    dim3 grid(n_seq, heads, slices);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(TO)                                                                                           \
    do {                                                                                                     \
        if (smem > 48 * 1024) {                                                                              \
            cudaError_t e = cudaFuncSetAttribute(ssd_scan_kernel<TO>,                                        \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
            if (e != cudaSuccess) return (int)e;                                                             \
        }                                                                                                    \
        RFX_LAUNCH(ssd_scan_kernel<TO>, grid, threads, smem, s, xbc, ldx, proj, ldp, z_off, dt_off, dt_bias, A, D, \
                   state, state_stride, state_off, seq_slot, seq_row0, (TO*)out, heads, P, N, groups, PW, KG); \
    } while (0)
    if (out_dt == RFX_DT_F32) RFX_GO(float);
    else if (out_dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}
