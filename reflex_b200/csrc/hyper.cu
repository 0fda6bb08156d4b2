// Hyper-connections: the residual as S parallel copies ("streams") of the
// model's width, 32-bit, [rows][S][W].
//
// A sublayer reads u = sum_s in[s] x_s and, with its result y (times a
// per-channel scale ls), every copy is rewritten at once from the old ones:
//     x_t <- sum_s mix[s][t] x_s + out[t] * (ls * y)        (mix is [from][to])
// S = 1 with in = out = mix = 1 is the ordinary residual sum x <- x + ls * y.
//
//  * rfx_hyper_expand: the embedding output into all S copies.
//  * rfx_hyper_step: the write of the sublayer before (if there is one), then the
//    read for the next sublayer and its RMS norm,
//        u / sqrt(mean(u^2) + eps) * (offset + w),
//    in one pass over the row: the copies are read once and written once, and
//    the norm needs no launch of its own.  A block owns a row; u stays in shared
//    memory between the sum of squares and the output.
//  * rfx_hyper_collapse: the last write and the sum of the copies, [rows][W].
//
// All arithmetic is 32-bit.  The sums over s run in index order.
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int MAX_S = 8;

struct Coef {
    float in[MAX_S];
    float out[MAX_S];
    float mix[MAX_S * MAX_S];
};

// the S new values of column c of a row: reads the old copies, applies the write
template <typename TY>
__device__ __forceinline__ void rewrite(const float* __restrict__ xrow, int S, int W, int c, const TY* __restrict__ yrow,
                                        const float* __restrict__ ls, const float* mix, const float* outw,
                                        float (&x)[MAX_S]) {
    float old[MAX_S];
#pragma unroll
    for (int s = 0; s < MAX_S; ++s) old[s] = s < S ? xrow[(size_t)s * W + c] : 0.0f;
    if (yrow == nullptr) {
#pragma unroll
        for (int s = 0; s < MAX_S; ++s) x[s] = old[s];
        return;
    }
    const float y = ls ? ld<TY>(yrow, c) * ls[c] : ld<TY>(yrow, c);
#pragma unroll
    for (int t = 0; t < MAX_S; ++t) {
        float v = 0.0f;
        if (t < S) {
            for (int s = 0; s < S; ++s) v = fmaf(mix[s * S + t], old[s], v);
            v = fmaf(outw[t], y, v);
        }
        x[t] = v;
    }
}

__global__ void __launch_bounds__(256)
hyper_expand_kernel(const float* __restrict__ x, float* __restrict__ streams, int S, int W) {
    pdl_prologue();
    const size_t r = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = x[r * W + c];
        for (int s = 0; s < S; ++s) streams[(r * S + s) * W + c] = v;
    }
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
hyper_step_kernel(float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ ls,
                  const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ in,
                  const float* __restrict__ norm_w, float eps, float w_offset, TO* __restrict__ out, int S, int W) {
    extern __shared__ float u_row[];  // [W]
    __shared__ float scratch[32];
    __shared__ Coef cf;
    pdl_launch_dependents();
    // the coefficients are weights: no kernel writes them
    if (threadIdx.x < S) {
        cf.in[threadIdx.x] = in[threadIdx.x];
        if (y) cf.out[threadIdx.x] = outw[threadIdx.x];
    }
    if (y && threadIdx.x < S * S) cf.mix[threadIdx.x] = mix[threadIdx.x];
    __syncthreads();
    pdl_wait();
    const size_t r = blockIdx.x;
    float* xrow = streams + r * S * W;
    const TY* yrow = y ? y + r * W : nullptr;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[MAX_S];
        rewrite<TY>(xrow, S, W, c, yrow, ls, cf.mix, cf.out, x);
        float u = 0.0f;
#pragma unroll
        for (int s = 0; s < MAX_S; ++s) {
            if (s < S) {
                if (yrow) xrow[(size_t)s * W + c] = x[s];
                u = fmaf(cf.in[s], x[s], u);
            }
        }
        u_row[c] = u;
        ss = fmaf(u, u, ss);
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(total / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        st<TO>(out, r * W + c, (u_row[c] * rinv) * (w_offset + norm_w[c]));
}

template <typename TY>
__global__ void __launch_bounds__(256)
hyper_collapse_kernel(const float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ ls,
                      const float* __restrict__ mix, const float* __restrict__ outw, float* __restrict__ out,
                      int S, int W) {
    __shared__ Coef cf;
    pdl_launch_dependents();
    if (y && threadIdx.x < S) cf.out[threadIdx.x] = outw[threadIdx.x];
    if (y && threadIdx.x < S * S) cf.mix[threadIdx.x] = mix[threadIdx.x];
    __syncthreads();
    pdl_wait();
    const size_t r = blockIdx.x;
    const float* xrow = streams + r * S * W;
    const TY* yrow = y ? y + r * W : nullptr;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        float x[MAX_S];
        rewrite<TY>(xrow, S, W, c, yrow, ls, cf.mix, cf.out, x);
        float sum = 0.0f;
#pragma unroll
        for (int s = 0; s < MAX_S; ++s)
            if (s < S) sum += x[s];
        out[r * W + c] = sum;
    }
}

}  // namespace

extern "C" int rfx_hyper_expand(const float* x, float* streams, int R, int S, int W, void* stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > MAX_S || W <= 0) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(hyper_expand_kernel, dim3(R), 256, 0, (cudaStream_t)stream, x, streams, S, W);
    return 0;
}

// `y` may be null (no write before the read); `ls` may be null (no per-channel scale).
extern "C" int rfx_hyper_step(float* streams, const void* y, int y_dt, const float* ls, const float* mix,
                              const float* outw, const float* in, const float* norm_w, float eps, float w_offset,
                              void* out, int out_dt, int R, int S, int W, void* stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > MAX_S || W <= 0 || (size_t)W * sizeof(float) > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    if (y && (!mix || !outw)) return RFX_ERR_BAD_ARG;
    const size_t smem = (size_t)W * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_HYPER(TY, TO)                                                                                          \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(hyper_step_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        RFX_LAUNCH((hyper_step_kernel<TY, TO>), dim3(R), 256, smem, s, streams, (const TY*)y, ls, mix, outw, in,   \
                   norm_w, eps, w_offset, (TO*)out, S, W);                                                         \
    } while (0)
    const bool y16 = y && y_dt == RFX_DT_BF16;
    if (out_dt == RFX_DT_F32) {
        if (y16) RFX_HYPER(__nv_bfloat16, float);
        else RFX_HYPER(float, float);
    } else if (out_dt == RFX_DT_BF16) {
        if (y16) RFX_HYPER(__nv_bfloat16, __nv_bfloat16);
        else RFX_HYPER(float, __nv_bfloat16);
    } else {
        return RFX_ERR_BAD_ARG;
    }
#undef RFX_HYPER
    return 0;
}

extern "C" int rfx_hyper_collapse(const float* streams, const void* y, int y_dt, const float* ls, const float* mix,
                                  const float* outw, float* out, int R, int S, int W, void* stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > MAX_S || W <= 0) return RFX_ERR_UNSUPPORTED;
    if (y && (!mix || !outw)) return RFX_ERR_BAD_ARG;
    int gy = (W + 255) / 256;
    if (R >= 64) gy = 1;
    else if (gy > 32) gy = 32;
    cudaStream_t s = (cudaStream_t)stream;
    if (y && y_dt == RFX_DT_BF16)
        RFX_LAUNCH(hyper_collapse_kernel<__nv_bfloat16>, dim3(R, gy), 256, 0, s, streams, (const __nv_bfloat16*)y, ls,
                   mix, outw, out, S, W);
    else
        RFX_LAUNCH(hyper_collapse_kernel<float>, dim3(R, gy), 256, 0, s, streams, (const float*)y, ls, mix, outw,
                   out, S, W);
    return 0;
}
