// Small row-wise ops around the residual stream, all with 32-bit arithmetic.
//
//  * rfx_branch_norm_mean: two branches' outputs, each over its root mean
//    square times its own weight, averaged:
//        out = ((a + a_bias) / rms(a + a_bias) * wa + b / rms(b) * wb) / 2
//  * rfx_glu_clamped: the clamped gated activation
//        g' = min(g, limit), u' = clamp(u, -limit, limit),
//        out = g' * sigmoid(alpha * g') * (u' + 1)
//    of a row [gates | ups] (or gate_j at 2j and up_j at 2j + 1).
//  * rfx_row_gate_add: y[r] += sigmoid(z[r]) * s[r] (+ extra[r]), one gate a row.
//  * rfx_stream_concat: out[r] = [x[r] (+ delta[r]) | x0[r]], cast, the input of
//    a product that mixes the stream with the embedding output.
//  * rfx_logit_finish: z <- z * scale, then cap * tanh(z / cap) when cap > 0.
#include "common.cuh"

namespace {

using namespace rfx;

// rows of up to PER * blockDim elements: a thread's elements stay in registers, all
// its loads are in flight together and global memory is read once
template <int PER>
__global__ void __launch_bounds__(1024)
branch_norm_mean_reg_kernel(const float* __restrict__ a, const float* __restrict__ a_bias,
                            const float* __restrict__ wa, const float* __restrict__ b,
                            const float* __restrict__ wb, float eps, float* __restrict__ out, int H) {
    __shared__ float scratch[32];
    pdl_prologue();
    const size_t r = blockIdx.x;
    float x[PER], y[PER];
    float sa = 0.0f, sb = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = i * blockDim.x + threadIdx.x;
        x[i] = c < H ? a[r * H + c] + (a_bias ? a_bias[c] : 0.0f) : 0.0f;
        y[i] = c < H ? b[r * H + c] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        sa = fmaf(x[i], x[i], sa);
        sb = fmaf(y[i], y[i], sb);
    }
    const float ra = rsqrtf(block_sum(sa, scratch) / (float)H + eps);
    const float rb = rsqrtf(block_sum(sb, scratch) / (float)H + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = i * blockDim.x + threadIdx.x;
        if (c < H) out[r * H + c] = 0.5f * fmaf(x[i] * ra, wa[c], (y[i] * rb) * wb[c]);
    }
}

__global__ void __launch_bounds__(256)
branch_norm_mean_kernel(const float* __restrict__ a, const float* __restrict__ a_bias,
                        const float* __restrict__ wa, const float* __restrict__ b,
                        const float* __restrict__ wb, float eps, float* __restrict__ out, int H) {
    __shared__ float scratch[32];
    pdl_prologue();
    const size_t r = blockIdx.x;
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = a[r * H + c] + (a_bias ? a_bias[c] : 0.0f);
        const float y = b[r * H + c];
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    const float ra = rsqrtf(block_sum(sa, scratch) / (float)H + eps);
    const float rb = rsqrtf(block_sum(sb, scratch) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = a[r * H + c] + (a_bias ? a_bias[c] : 0.0f);
        const float y = b[r * H + c];
        out[r * H + c] = 0.5f * fmaf(x * ra, wa[c], (y * rb) * wb[c]);
    }
}

__device__ __forceinline__ float glu_clamped(float g, float u, float alpha, float limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int R, int I, int alternating,
                                   float alpha, float limit) {
    pdl_prologue();
    const size_t n = (size_t)R * I;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / I, c = i % I;
        const float g = ld<T>(gu, r * 2 * I + (alternating ? 2 * c : c));
        const float u = ld<T>(gu, r * 2 * I + (alternating ? 2 * c + 1 : I + c));
        st<T>(out, i, glu_clamped(g, u, alpha, limit));
    }
}

// bfloat16, I a multiple of 8, 16-byte aligned rows: eight outputs a thread and step
__global__ void __launch_bounds__(256)
glu_clamped_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int R, int I,
                          int alternating, float alpha, float limit) {
    pdl_prologue();
    const size_t n8 = (size_t)R * (I / 8);
    const unsigned i8 = (unsigned)(I / 8);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 *pa, *pb;
        if (alternating) {  // output pack i comes from input elements [16 i, 16 i + 16)
            pa = reinterpret_cast<const uint4*>(gu + 16 * i);
            pb = pa + 1;
        } else {
            const size_t r = i / i8, c = (i - r * i8) * 8;
            pa = reinterpret_cast<const uint4*>(gu + r * 2 * I + c);
            pb = reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c);
        }
        const uint4 a = *pa, b = *pb;
        const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
        if (alternating) {  // a = g0 u0 g1 u1 g2 u2 g3 u3, b = g4 u4 ...
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float2 p0 = __bfloat1622float2(ha[2 * j]), p1 = __bfloat1622float2(ha[2 * j + 1]);
                const float2 q0 = __bfloat1622float2(hb[2 * j]), q1 = __bfloat1622float2(hb[2 * j + 1]);
                ho[j] = __floats2bfloat162_rn(glu_clamped(p0.x, p0.y, alpha, limit), glu_clamped(p1.x, p1.y, alpha, limit));
                ho[2 + j] = __floats2bfloat162_rn(glu_clamped(q0.x, q0.y, alpha, limit),
                                                  glu_clamped(q1.x, q1.y, alpha, limit));
            }
        } else {  // a = eight gates, b = their ups
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 g = __bfloat1622float2(ha[j]), up = __bfloat1622float2(hb[j]);
                ho[j] = __floats2bfloat162_rn(glu_clamped(g.x, up.x, alpha, limit), glu_clamped(g.y, up.y, alpha, limit));
            }
        }
        *reinterpret_cast<uint4*>(out + 8 * i) = o;
    }
}

template <typename T>
__global__ void row_gate_add_kernel(float* __restrict__ y, const T* __restrict__ s, const float* __restrict__ z,
                                    int ldz, int col, const float* __restrict__ extra, int H) {
    pdl_prologue();
    const size_t r = blockIdx.x;
    const float gate = 1.0f / (1.0f + expf(-z[r * ldz + col]));
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x) {
        float v = y[r * H + c];
        if (extra) v += extra[r * H + c];
        y[r * H + c] = fmaf(gate, ld<T>(s, r * H + c), v);
    }
}

template <typename TD, typename TO>
__global__ void stream_concat_kernel(const float* __restrict__ x, const TD* __restrict__ delta,
                                     const float* __restrict__ x0, TO* __restrict__ out, int H) {
    pdl_prologue();
    const size_t r = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x) {
        float v = x[r * H + c];
        if (delta) v += ld<TD>(delta, r * H + c);
        st<TO>(out, r * 2 * H + c, v);
        st<TO>(out, r * 2 * H + H + c, x0[r * H + c]);
    }
}

__global__ void logit_finish_kernel(float* __restrict__ z, size_t n, float scale, float cap) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = z[i] * scale;
        if (cap > 0.0f) v = cap * tanhf(v / cap);
        z[i] = v;
    }
}

// a[r][c] <- a[r][c] * sigmoid(z[r][col + c]): a gate computed beside the values it
// scales (columns of the same stacked product); the sigmoid is 32-bit
template <typename TA, typename TZ>
__global__ void __launch_bounds__(256)
sigmoid_gate_mul_kernel(TA* __restrict__ a, const TZ* __restrict__ z, int ldz, int col, int H) {
    pdl_prologue();
    const size_t r = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H; c += gridDim.y * blockDim.x) {
        const float g = ld<TZ>(z, r * ldz + col + c);
        st<TA>(a, r * H + c, ld<TA>(a, r * H + c) / (1.0f + expf(-g)));
    }
}

// the same for bfloat16 `a`, four neighbouring elements a thread (8-byte accesses of `a`, 8 or
// 16 of `z`); H, ldz and col multiples of four
template <typename TZ>
__global__ void __launch_bounds__(256)
sigmoid_gate_mul4_kernel(__nv_bfloat16* __restrict__ a, const TZ* __restrict__ z, int ldz, int col, int H) {
    pdl_prologue();
    const size_t r = blockIdx.x;
    for (int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x); c < H; c += 4 * gridDim.y * blockDim.x) {
        float g[4];
        if constexpr (sizeof(TZ) == 4) {
            const float4 v = *reinterpret_cast<const float4*>(z + r * ldz + col + c);
            g[0] = v.x, g[1] = v.y, g[2] = v.z, g[3] = v.w;
        } else {
            const uint2 v = *reinterpret_cast<const uint2*>(z + r * ldz + col + c);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            g[0] = lo.x, g[1] = lo.y, g[2] = hi.x, g[3] = hi.y;
        }
        uint2 av = *reinterpret_cast<const uint2*>(a + r * H + c);
        float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av.x));
        float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av.y));
        a0.x = a0.x / (1.0f + expf(-g[0]));
        a0.y = a0.y / (1.0f + expf(-g[1]));
        a1.x = a1.x / (1.0f + expf(-g[2]));
        a1.y = a1.y / (1.0f + expf(-g[3]));
        *reinterpret_cast<__nv_bfloat162*>(&av.x) = __floats2bfloat162_rn(a0.x, a0.y);
        *reinterpret_cast<__nv_bfloat162*>(&av.y) = __floats2bfloat162_rn(a1.x, a1.y);
        *reinterpret_cast<uint2*>(a + r * H + c) = av;
    }
}

// blocks along a row for kernels that take a row's elements independently: few rows get a
// thread an element (every load in flight at once), many rows walk their row
int row_chunks(int R, int H) {
    int g = (H + 255) / 256;
    const int most = sm_count() * 8 / (R < 1 ? 1 : R);
    if (g > most) g = most;
    return g < 1 ? 1 : g;
}

int blocks_for(size_t n) {
    size_t b = (n + 255) / 256;
    const size_t most = (size_t)sm_count() * 16;
    return (int)(b > most ? most : (b < 1 ? 1 : b));
}

}  // namespace

extern "C" int rfx_branch_norm_mean(const float* a, const float* a_bias, const float* wa, const float* b,
                                    const float* wb, float eps, float* out, int R, int H, void* stream) {
    if (R <= 0 || H <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (H <= 4 * 128) RFX_LAUNCH(branch_norm_mean_reg_kernel<4>, R, 128, 0, s, a, a_bias, wa, b, wb, eps, out, H);
    else if (H <= 4 * 256) RFX_LAUNCH(branch_norm_mean_reg_kernel<4>, R, 256, 0, s, a, a_bias, wa, b, wb, eps, out, H);
    else if (H <= 4 * 512) RFX_LAUNCH(branch_norm_mean_reg_kernel<4>, R, 512, 0, s, a, a_bias, wa, b, wb, eps, out, H);
    else if (H <= 8 * 1024) RFX_LAUNCH(branch_norm_mean_reg_kernel<8>, R, 1024, 0, s, a, a_bias, wa, b, wb, eps, out, H);
    else RFX_LAUNCH(branch_norm_mean_kernel, R, 256, 0, s, a, a_bias, wa, b, wb, eps, out, H);
    return 0;
}

extern "C" int rfx_glu_clamped(const void* gate_up, void* out, int dt, int R, int I, int alternating,
                               float alpha, float limit, void* stream) {
    if (R <= 0 || I <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = blocks_for((size_t)R * I);
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(glu_clamped_kernel<float>, blocks, 256, 0, s, (const float*)gate_up, (float*)out, R, I,
                   alternating, alpha, limit);
    else if (dt == RFX_DT_BF16 && I % 8 == 0 &&
             ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
        RFX_LAUNCH(glu_clamped_bf16x8_kernel, blocks_for((size_t)R * I / 8), 256, 0, s,
                   (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, R, I, alternating, alpha, limit);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(glu_clamped_kernel<__nv_bfloat16>, blocks, 256, 0, s, (const __nv_bfloat16*)gate_up,
                   (__nv_bfloat16*)out, R, I, alternating, alpha, limit);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_row_gate_add(float* y, const void* s_rows, int dt, const float* z, int ldz, int col,
                                const float* extra, int R, int H, void* stream) {
    if (R <= 0 || H <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(row_gate_add_kernel<float>, dim3(R, row_chunks(R, H)), 256, 0, s, y, (const float*)s_rows, z, ldz,
                   col, extra, H);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(row_gate_add_kernel<__nv_bfloat16>, dim3(R, row_chunks(R, H)), 256, 0, s, y,
                   (const __nv_bfloat16*)s_rows, z, ldz, col, extra, H);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_stream_concat(const float* x, const void* delta, int delta_dt, const float* x0, void* out,
                                 int out_dt, int R, int H, void* stream) {
    if (R <= 0 || H <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool dbf = delta && delta_dt == RFX_DT_BF16;
    if (delta && delta_dt != RFX_DT_BF16 && delta_dt != RFX_DT_F32) return RFX_ERR_BAD_ARG;
#define RFX_GO(TD, TO)                                                                                   \
    RFX_LAUNCH((stream_concat_kernel<TD, TO>), dim3(R, row_chunks(R, H)), 256, 0, s, x, (const TD*)delta, x0, \
               (TO*)out, H)
    if (out_dt == RFX_DT_F32) {
        if (dbf) RFX_GO(__nv_bfloat16, float);
        else RFX_GO(float, float);
    } else if (out_dt == RFX_DT_BF16) {
        if (dbf) RFX_GO(__nv_bfloat16, __nv_bfloat16);
        else RFX_GO(float, __nv_bfloat16);
    } else
        return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}

extern "C" int rfx_logit_finish(float* z, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return 0;
    RFX_LAUNCH(logit_finish_kernel, blocks_for((size_t)n), 256, 0, (cudaStream_t)stream, z, (size_t)n, scale,
               cap);
    return 0;
}

extern "C" int rfx_sigmoid_gate_mul(void* a, int a_dt, const void* z, int z_dt, int ldz, int col, int R, int H,
                                    void* stream) {
    if (R <= 0 || H <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(R, row_chunks(R, H));
    const bool by4 = a_dt == RFX_DT_BF16 && H % 4 == 0 && ldz % 4 == 0 && col % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(a) & 7) == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0;
    if (by4 && (z_dt == RFX_DT_F32 || z_dt == RFX_DT_BF16)) {
        const dim3 grid4(R, row_chunks(R, H / 4));
        if (z_dt == RFX_DT_F32)
            RFX_LAUNCH(sigmoid_gate_mul4_kernel<float>, grid4, 256, 0, s, (__nv_bfloat16*)a, (const float*)z, ldz, col, H);
        else
            RFX_LAUNCH(sigmoid_gate_mul4_kernel<__nv_bfloat16>, grid4, 256, 0, s, (__nv_bfloat16*)a,
                       (const __nv_bfloat16*)z, ldz, col, H);
        return 0;
    }
    if (a_dt == RFX_DT_F32 && z_dt == RFX_DT_F32)
        RFX_LAUNCH((sigmoid_gate_mul_kernel<float, float>), grid, 256, 0, s, (float*)a, (const float*)z, ldz, col, H);
    else if (a_dt == RFX_DT_BF16 && z_dt == RFX_DT_F32)
        RFX_LAUNCH((sigmoid_gate_mul_kernel<__nv_bfloat16, float>), grid, 256, 0, s, (__nv_bfloat16*)a,
                   (const float*)z, ldz, col, H);
    else if (a_dt == RFX_DT_BF16 && z_dt == RFX_DT_BF16)
        RFX_LAUNCH((sigmoid_gate_mul_kernel<__nv_bfloat16, __nv_bfloat16>), grid, 256, 0, s, (__nv_bfloat16*)a,
                   (const __nv_bfloat16*)z, ldz, col, H);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
