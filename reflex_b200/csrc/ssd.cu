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
// Two forms.  The one below the general one takes channel and state counts that are
// multiples of four, up to 256 states (see there).  The general one:
// a block owns (sequence, head, slice of the P channels) and walks the
// sequence's rows in order; its part of S lives in shared memory; thread
// (k, p) takes the states n = k, k + KG, ... of channel p, and the KG partial
// sums of y meet in shared memory in index order, so a row's result does not
// depend on how the work was cut into steps or on what else is in the batch.
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


// ---- the form for channel and state counts that are multiples of four -------------
// A block owns (sequence, head, some of the channels) and walks the rows in tiles of
// TT: all its threads first stage a tile (B, C, x and z of its rows, 16 bytes a load,
// their step sizes and decays into shared memory), then each warp walks the tile's
// rows on its own channels (four, two or one) with no further barrier: KG lanes (8, 16 or
// 32) share a channel, lane (g, c) holds its states 4 (g + KG m) .. + 3 in registers (NC
// groups of four, B and C read from the tile 16 bytes at a time), the KG partial sums of y
// meet by shuffles.  The
// state lies [heads][channel][state].  Which block and warp walks a channel changes
// nothing of its arithmetic.
template <int NC, int KG, typename TO>
__global__ void __launch_bounds__(512)
ssd_scan_warp_kernel(const float* __restrict__ xbc, int ldx, const float* __restrict__ proj, int ldp, int z_off,
                     int dt_off, const float* __restrict__ dt_bias, const float* __restrict__ A,
                     const float* __restrict__ D, float* __restrict__ state, long long state_stride,
                     long long state_off, const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                     TO* __restrict__ out, int heads, int P, int N, int groups, int cols, int TT) {
    extern __shared__ __align__(16) float sm[];  // [TT][2 N + 2 cols + 4]: B, C, x, silu(z), dt, decay
    pdl_prologue();
    const int seq = blockIdx.x, h = blockIdx.y, c_first = blockIdx.z * cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int CW = 32 / KG;  // channels a warp walks; KG lanes share a channel
    const int g = lane / CW, cl = warp * CW + (lane % CW), col = c_first + cl;
    const int grp = h / (heads / groups);
    const int inner = heads * P, N4 = N / 4, c4 = cols / 4;
    const int row0 = seq_row0[seq], row1 = seq_row0[seq + 1];
    const int stride = 2 * N + 2 * cols + 4, stride4 = stride / 4;
    float* Sg = state + (size_t)seq_slot[seq] * state_stride + state_off + ((size_t)h * P + col) * N;
    float S[NC][4];
#pragma unroll
    for (int m = 0; m < NC; ++m)
#pragma unroll
        for (int q = 0; q < 4; ++q) S[m][q] = g + KG * m < N4 ? Sg[4 * (g + KG * m) + q] : 0.0f;
    const float a = A[h], dcoef = D ? D[h] : 0.0f, bias = dt_bias ? dt_bias[h] : 0.0f;
    float4* sm4 = reinterpret_cast<float4*>(sm);
    for (int t0 = row0; t0 < row1; t0 += TT) {
        const int nt = min(TT, row1 - t0);
        __syncthreads();  // the tile before has been walked by every warp
        const float* xr0 = xbc + (size_t)t0 * ldx;
        const float* pr0 = proj + (size_t)t0 * ldp;
#pragma unroll 4
        for (int e = threadIdx.x; e < nt * 2 * N4; e += blockDim.x) {  // B and C
            const int t = e / (2 * N4), c = e - t * 2 * N4;
            const int src = c < N4 ? inner + grp * N + 4 * c : inner + groups * N + grp * N + 4 * (c - N4);
            sm4[(size_t)t * stride4 + c] = *reinterpret_cast<const float4*>(xr0 + (size_t)t * ldx + src);
        }
#pragma unroll 4
        for (int e = threadIdx.x; e < nt * c4; e += blockDim.x) {  // x and z
            const int t = e / c4, c = e - t * c4;
            const float4 xv = *reinterpret_cast<const float4*>(xr0 + (size_t)t * ldx + h * P + c_first + 4 * c);
            const float4 zv = *reinterpret_cast<const float4*>(pr0 + (size_t)t * ldp + z_off + h * P + c_first + 4 * c);
            sm4[(size_t)t * stride4 + 2 * N4 + c] = xv;
            // the gate silu(z), made once an element here
            sm4[(size_t)t * stride4 + 2 * N4 + c4 + c] =
                make_float4(zv.x / (1.0f + expf(-zv.x)), zv.y / (1.0f + expf(-zv.y)), zv.z / (1.0f + expf(-zv.z)),
                            zv.w / (1.0f + expf(-zv.w)));
        }
        for (int t = threadIdx.x; t < nt; t += blockDim.x) {  // the rows' step sizes and decays
            const float dt = softplus_f(pr0[(size_t)t * ldp + dt_off + h] + bias);
            sm[(size_t)t * stride + 2 * N + 2 * cols] = dt;
            sm[(size_t)t * stride + 2 * N + 2 * cols + 1] = expf(a * dt);
        }
        __syncthreads();
        // four rows at a time: the state's steps follow one another, the rows' partial sums of y
        // meet by shuffles together (their chains run side by side), then the rows are written
        for (int t = 0; t < nt; t += 4) {
            float yv[4], xs[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                yv[u] = 0.0f;
                xs[u] = 0.0f;
                if (t + u < nt) {
                    const float* tile = sm + (size_t)(t + u) * stride;
                    const float4* tile4 = reinterpret_cast<const float4*>(tile);
                    const float x = tile[2 * N + cl], decay = tile[2 * N + 2 * cols + 1];
                    const float dx = tile[2 * N + 2 * cols] * x;
                    float y = 0.0f, y1 = 0.0f;
#pragma unroll
                    for (int m = 0; m < NC; ++m) {
                        const int c = g + KG * m;
                        if (c < N4) {
                            const float4 b = tile4[c], cc = tile4[N4 + c];
                            S[m][0] = fmaf(S[m][0], decay, b.x * dx);
                            S[m][1] = fmaf(S[m][1], decay, b.y * dx);
                            S[m][2] = fmaf(S[m][2], decay, b.z * dx);
                            S[m][3] = fmaf(S[m][3], decay, b.w * dx);
                            y = fmaf(S[m][0], cc.x, fmaf(S[m][1], cc.y, y));
                            y1 = fmaf(S[m][2], cc.z, fmaf(S[m][3], cc.w, y1));
                        }
                    }
                    yv[u] = y + y1;
                    xs[u] = x;
                }
            }
#pragma unroll
            for (int off = CW; off < 32; off <<= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) yv[u] += __shfl_xor_sync(0xffffffffu, yv[u], off);
            if (g == 0) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (t + u < nt) {
                        const float gate = sm[(size_t)(t + u) * stride + 2 * N + cols + cl];  // silu(z)
                        st<TO>(out, (size_t)(t0 + t + u) * inner + h * P + col, fmaf(dcoef, xs[u], yv[u]) * gate);
                    }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < NC; ++m)
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (g + KG * m < N4) Sg[4 * (g + KG * m) + q] = S[m][q];
}

template <int NC, int KG, typename TO>
int launch_warp(const float* xbc, int ldx, const float* proj, int ldp, int z_off, int dt_off, const float* dt_bias,
                const float* A, const float* D, float* state, long long state_stride, long long state_off,
                const int* seq_slot, const int* seq_row0, int n_seq, void* out, int heads, int P, int N, int groups,
                cudaStream_t s) {
    // channels a block owns (four a warp): the largest divisor of P that is a multiple of
    // four and at most 64; fewer while the blocks do not fill the SMs
    constexpr int CW = 32 / KG;  // channels a warp
    // (a multiple of four: x and z are staged 16 bytes a load)
    int cols = 0;
    for (int c = 4; c <= 16 * CW && c <= P; c += 4)
        if (P % c == 0) cols = c;
    if (!cols) return RFX_ERR_UNSUPPORTED;
    while (cols % 8 == 0 && cols > scan_min_warps() * CW && cols > 4 && (long long)n_seq * heads * (P / cols) < sm_count())
        cols /= 2;
    const int stride = 2 * N + 2 * cols + 4;
    int TT = (48 * 1024) / (stride * (int)sizeof(float));
    if (TT > 32) TT = 32;
    if (TT < 1) TT = 1;
    const size_t smem = (size_t)TT * stride * sizeof(float);
    auto kernel = ssd_scan_warp_kernel<NC, KG, TO>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_seq, heads, P / cols);
    RFX_LAUNCH(kernel, grid, (cols / CW) * 32, smem, s, xbc, ldx, proj, ldp, z_off, dt_off, dt_bias, A, D, state,
               state_stride, state_off, seq_slot, seq_row0, (TO*)out, heads, P, N, groups, cols, TT);
    return 0;
}

}  // namespace

extern "C" int rfx_ssd_scan(const float* xbc, int ldx, const float* proj, int ldp, int z_off, int dt_off,
                            const float* dt_bias, const float* A, const float* D, float* state,
                            long long state_stride, long long state_off, const int* seq_slot, const int* seq_row0,
                            int n_seq, void* out, int out_dt, int heads, int P, int N, int groups, void* stream) {
    if (n_seq <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0) return RFX_ERR_BAD_ARG;
    const bool aligned = ((ldx | ldp | z_off) & 3) == 0 &&
                         ((reinterpret_cast<uintptr_t>(xbc) | reinterpret_cast<uintptr_t>(proj)) & 15) == 0;
    if (P % 4 == 0 && N % 4 == 0 && N <= 256 && out_dt == RFX_DT_F32 && aligned) {
#define RFX_WARP(NP, G)                                                                                   \
    st = launch_warp<NP, G, float>(xbc, ldx, proj, ldp, z_off, dt_off, dt_bias, A, D, state, state_stride, \
                                   state_off, seq_slot, seq_row0, n_seq, out, heads, P, N, groups,         \
                                   (cudaStream_t)stream)
        int st;  // a channel count that does not divide among the warps goes to the general form
        // as many lanes a channel as it has groups of four states (8, 16 or 32): a lane's share is one
        // or two groups, and a head gives enough warps to keep the SMs' schedulers busy
        if (N <= 32) RFX_WARP(1, 8);
        else if (N <= 64) RFX_WARP(1, 16);
        else if (N <= 128) RFX_WARP(1, 32);
        else RFX_WARP(2, 32);
        if (st != RFX_ERR_UNSUPPORTED) return st;
#undef RFX_WARP
    }
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
