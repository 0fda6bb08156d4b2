// Row-wise kernels of layers that norm a sublayer's result before it joins the
// residual (a norm on both sides of every sublayer), and a few small companions.
//
// sandwich_norm: with y a sublayer's 32-bit result [R, H], the residual x [R, H]
// (32-bit, updated in place) and two weights,
//     x <- x + mult * y * rsqrt(mean(y^2) + eps) * w_post
//     out = x * rsqrt(mean(x^2) + eps) * w_next        (when w_next is given)
// so the norm after one sublayer and the norm before the next are one pass over
// the row.  A block a row; the row lives in shared memory between the sums of
// squares and the outputs.
//
// group_norm_gate: x [R, C] 32-bit in `groups` equal parts, each over its own
// root mean square, times w[c], times sigmoid(z[r, col + c]) when a gate is given.
//
// xielu: z > 0: ap z^2 + z / 2; else an (e^z - 1 - z) + z / 2, with ap and an given
// (the softplus of the stored numbers is taken once, when the weights are bound).
//
// loop_input: x[r, :] += x0[r, :] (when given) + vec[:], the start of a pass over
// a repeated stretch of layers.  tanh_cols: out[r, j] = tanh(in[r, col + j]).
// scaled_sum: a <- sa * a + sb * b.
#include "common.cuh"

namespace {

using namespace rfx;

template <typename TO>
__global__ void __launch_bounds__(256)
sandwich_norm_kernel(const float* __restrict__ y, float* __restrict__ x, const float* __restrict__ w_post,
                     float mult, float eps, const float* __restrict__ w_next, float eps_next,
                     TO* __restrict__ out, int H) {
    extern __shared__ __align__(16) float row[];  // [H]
    __shared__ float scratch[32];
    pdl_prologue();
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = y[base + c];
        row[c] = v;
        ss = fmaf(v, v, ss);
    }
    const float r1 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = fmaf(mult, (row[c] * r1) * w_post[c], x[base + c]);
        x[base + c] = v;
        row[c] = v;
        ss = fmaf(v, v, ss);
    }
    if (w_next == nullptr) return;
    const float r2 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps_next);
    for (int c = threadIdx.x; c < H; c += blockDim.x) st<TO>(out, base + c, (row[c] * r2) * w_next[c]);
}

// The same with 16-byte accesses, for widths that are a multiple of four: the row stays in
// registers (up to V groups of four a thread) between the sums of squares and the outputs.
template <typename TO, int V>
__global__ void __launch_bounds__(512)
sandwich_norm4_kernel(const float* __restrict__ y, float* __restrict__ x, const float* __restrict__ w_post,
                      float mult, float eps, const float* __restrict__ w_next, float eps_next,
                      TO* __restrict__ out, int H) {
    __shared__ float scratch[32];
    pdl_prologue();
    const size_t base = (size_t)blockIdx.x * H;
    const int H4 = H / 4;
    const float4* y4 = reinterpret_cast<const float4*>(y + base);
    float4* x4 = reinterpret_cast<float4*>(x + base);
    const float4* wp4 = reinterpret_cast<const float4*>(w_post);
    float4 v[V], xv[V], wp[V];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < H4) {
            v[i] = y4[c];
            xv[i] = x4[c];
            wp[i] = wp4[c];
            ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
        }
    }
    const float r1 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    ss = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < H4) {
            v[i].x = fmaf(mult, (v[i].x * r1) * wp[i].x, xv[i].x);
            v[i].y = fmaf(mult, (v[i].y * r1) * wp[i].y, xv[i].y);
            v[i].z = fmaf(mult, (v[i].z * r1) * wp[i].z, xv[i].z);
            v[i].w = fmaf(mult, (v[i].w * r1) * wp[i].w, xv[i].w);
            x4[c] = v[i];
            ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
        }
    }
    if (w_next == nullptr) return;
    const float r2 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps_next);
    const float4* wn4 = reinterpret_cast<const float4*>(w_next);
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < H4) {
            const float4 wn = wn4[c];
            store4(out + base + 4 * (size_t)c, make_float4((v[i].x * r2) * wn.x, (v[i].y * r2) * wn.y,
                                                           (v[i].z * r2) * wn.z, (v[i].w * r2) * wn.w));
        }
    }
}

// One block a (row, part), 16 bytes an access: parts of many elements (a norm in a few equal
// parts of a wide row), where a warp a part would leave a row to a warp or two.
template <typename TO>
__global__ void __launch_bounds__(256)
group_norm_gate_wide_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                            const float* __restrict__ z, int ldz, int zcol, TO* __restrict__ out, int C, int gs) {
    __shared__ float scratch[32];
    pdl_prologue();
    const int r = blockIdx.x, g = blockIdx.y;
    const size_t base = (size_t)r * C + (size_t)g * gs;
    const float4* x4 = reinterpret_cast<const float4*>(x + base);
    const float4* w4 = reinterpret_cast<const float4*>(w + (size_t)g * gs);
    float ss = 0.0f;
    for (int c = threadIdx.x; c < gs / 4; c += blockDim.x) {
        const float4 v = x4[c];
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    const float rs = 1.0f / sqrtf(block_sum(ss, scratch) / (float)gs + eps);
    for (int c = threadIdx.x; c < gs / 4; c += blockDim.x) {
        const float4 v = x4[c], wv = w4[c];
        float4 o = make_float4((v.x * rs) * wv.x, (v.y * rs) * wv.y, (v.z * rs) * wv.z, (v.w * rs) * wv.w);
        if (z) {
            const float* zp = z + (size_t)r * ldz + zcol + (size_t)g * gs + 4 * c;
            o.x *= 1.0f / (1.0f + exact_expf(-zp[0]));
            o.y *= 1.0f / (1.0f + exact_expf(-zp[1]));
            o.z *= 1.0f / (1.0f + exact_expf(-zp[2]));
            o.w *= 1.0f / (1.0f + exact_expf(-zp[3]));
        }
        store4(out + base + 4 * (size_t)c, o);
    }
}

template <typename TO>
__global__ void __launch_bounds__(256)
group_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                       const float* __restrict__ z, int ldz, int zcol, TO* __restrict__ out, int C, int groups) {
    pdl_prologue();
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int gs = C / groups;
    // a warp a part; a row's parts spread over the blocks of its grid row
    for (int g = blockIdx.y * nwarps + warp; g < groups; g += gridDim.y * nwarps) {
        const float* xr = x + (size_t)r * C + (size_t)g * gs;
        float ss = 0.0f;
        for (int c = lane; c < gs; c += 32) ss = fmaf(xr[c], xr[c], ss);
        const float rs = 1.0f / sqrtf(warp_sum(ss) / (float)gs + eps);
        for (int c = lane; c < gs; c += 32) {
            float v = (xr[c] * rs) * w[g * gs + c];
            if (z) {
                const float t = z[(size_t)r * ldz + zcol + g * gs + c];
                v *= 1.0f / (1.0f + exact_expf(-t));
            }
            st<TO>(out, (size_t)r * C + (size_t)g * gs + c, v);
        }
    }
}

template <typename T>
__global__ void xielu_kernel(T* __restrict__ a, size_t n, float ap, float an) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float z = ld<T>(a, i);
        float v;
        if (z > 0.0f) v = fmaf(ap * z, z, 0.5f * z);
        else v = fmaf(an, expm1f(z) - z, 0.5f * z);
        st<T>(a, i, v);
    }
}

__global__ void loop_input_kernel(float* __restrict__ x, const float* __restrict__ x0,
                                  const float* __restrict__ vec, size_t n, int H) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (x0) v += x0[i];
        x[i] = v + vec[i % H];
    }
}

template <typename TO>
__global__ void tanh_cols_kernel(const float* __restrict__ in, int ld, int col, TO* __restrict__ out, int R, int n) {
    pdl_prologue();
    const size_t total = (size_t)R * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        st<TO>(out, i, tanhf(in[(i / n) * ld + col + (i % n)]));
}

__global__ void scaled_sum_kernel(float* __restrict__ a, const float* __restrict__ b, float sa, float sb, size_t n) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        a[i] = fmaf(sa, a[i], sb * b[i]);
}

inline int blocks_for(size_t n, int threads) {
    size_t b = (n + threads - 1) / threads;
    const size_t cap = (size_t)sm_count() * 8;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

extern "C" int rfx_sandwich_norm(const float* y, float* x, const float* w_post, float mult, float eps,
                                 const float* w_next, float eps_next, void* out, int out_dt, int R, int H,
                                 void* stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const bool al = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_post) |
                      reinterpret_cast<uintptr_t>(w_next) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (H % 4 == 0 && H <= 4 * 512 * 4 && al) {
        // the row in registers, 16 bytes an access; threads so that a thread holds one to four groups
        const int H4 = H / 4;
        const int threads = H4 <= 128 ? 128 : H4 <= 256 ? 256 : 512;
#define RFX_V(TO, V)                                                                                           \
    RFX_LAUNCH((sandwich_norm4_kernel<TO, V>), R, threads, 0, s, y, x, w_post, mult, eps, w_next, eps_next,   \
               (TO*)out, H)
#define RFX_PICK(TO)                                      \
    do {                                                  \
        if (H4 <= threads) RFX_V(TO, 1);                  \
        else if (H4 <= 2 * threads) RFX_V(TO, 2);         \
        else RFX_V(TO, 4);                                \
    } while (0)
        if (out_dt == RFX_DT_F32) RFX_PICK(float);
        else if (out_dt == RFX_DT_BF16) RFX_PICK(__nv_bfloat16);
        else return RFX_ERR_BAD_ARG;
#undef RFX_PICK
#undef RFX_V
        return 0;
    }
#define RFX_GO(TO)                                                                                          \
    do {                                                                                                    \
        if (smem > 48 * 1024) {                                                                             \
            cudaError_t e = cudaFuncSetAttribute(sandwich_norm_kernel<TO>,                                  \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
            if (e != cudaSuccess) return (int)e;                                                            \
        }                                                                                                   \
        RFX_LAUNCH(sandwich_norm_kernel<TO>, R, 256, smem, s, y, x, w_post, mult, eps, w_next, eps_next,    \
                   (TO*)out, H);                                                                            \
    } while (0)
    if (out_dt == RFX_DT_F32) RFX_GO(float);
    else if (out_dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}

extern "C" int rfx_group_norm_gate(const float* x, const float* w, float eps, const float* z, int ldz, int zcol,
                                   void* out, int out_dt, int R, int C, int groups, void* stream) {
    if (R <= 0) return 0;
    if (groups <= 0 || C % groups) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int gs = C / groups;
    const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (gs >= 512 && gs % 4 == 0 && C % 4 == 0 && al && groups <= 65535) {
        dim3 grid(R, groups);
        if (out_dt == RFX_DT_F32)
            RFX_LAUNCH(group_norm_gate_wide_kernel<float>, grid, 256, 0, s, x, w, eps, z, ldz, zcol, (float*)out, C, gs);
        else if (out_dt == RFX_DT_BF16)
            RFX_LAUNCH(group_norm_gate_wide_kernel<__nv_bfloat16>, grid, 256, 0, s, x, w, eps, z, ldz, zcol,
                       (__nv_bfloat16*)out, C, gs);
        else return RFX_ERR_BAD_ARG;
        return 0;
    }
    const int threads = groups >= 4 ? 128 : 32 * groups;
    int gy = (groups + 3) / 4;
    if (gy > 65535) gy = 65535;
    dim3 grid(R, gy);
    if (out_dt == RFX_DT_F32)
        RFX_LAUNCH(group_norm_gate_kernel<float>, grid, threads, 0, s, x, w, eps, z, ldz, zcol, (float*)out, C, groups);
    else if (out_dt == RFX_DT_BF16)
        RFX_LAUNCH(group_norm_gate_kernel<__nv_bfloat16>, grid, threads, 0, s, x, w, eps, z, ldz, zcol,
                   (__nv_bfloat16*)out, C, groups);
    else return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_xielu(void* a, int dt, long long n, float ap, float an, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = blocks_for((size_t)n, 256);
    if (dt == RFX_DT_F32) RFX_LAUNCH(xielu_kernel<float>, blocks, 256, 0, s, (float*)a, (size_t)n, ap, an);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(xielu_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)a, (size_t)n, ap, an);
    else return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_loop_input(float* x, const float* x0, const float* vec, int R, int H, void* stream) {
    if (R <= 0) return 0;
    const size_t n = (size_t)R * H;
    RFX_LAUNCH(loop_input_kernel, blocks_for(n, 256), 256, 0, (cudaStream_t)stream, x, x0, vec, n, H);
    return 0;
}

extern "C" int rfx_tanh_cols(const float* in, int ld, int col, void* out, int out_dt, int R, int n, void* stream) {
    if (R <= 0 || n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = blocks_for((size_t)R * n, 256);
    if (out_dt == RFX_DT_F32) RFX_LAUNCH(tanh_cols_kernel<float>, blocks, 256, 0, s, in, ld, col, (float*)out, R, n);
    else if (out_dt == RFX_DT_BF16)
        RFX_LAUNCH(tanh_cols_kernel<__nv_bfloat16>, blocks, 256, 0, s, in, ld, col, (__nv_bfloat16*)out, R, n);
    else return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_scaled_sum(float* a, const float* b, float sa, float sb, long long n, void* stream) {
    if (n <= 0) return 0;
    RFX_LAUNCH(scaled_sum_kernel, blocks_for((size_t)n, 256), 256, 0, (cudaStream_t)stream, a, b, sa, sb, (size_t)n);
    return 0;
}
