// Block-diagonal product: the columns of a row are cut into B equal parts and part b goes through a matrix of
// its own,
//   out[t, b*N + n] = epi( sum_k x[t, b*K + k] * W[b, n, k] + bias[b*N + n] ),   W: [B, N, K]
// This is one product per head of an attention layer (queries taken into the key latent, the latent result
// taken up to values) and the gates of a recurrence whose gate matrices are block-diagonal.
//   epi 0  nothing
//   epi 1  sigmoid(.)
//   epi 2  (.) * sigmoid(gate[t, b*N + n])      gate: float rows with a stride of their own
// Three kernels, all with float accumulation and with an output element's sum depending on nothing but its own
// row (not on the step's other rows or their number):
//   tiles on the CUDA cores: any sizes, strides and types (the float32 path; the fallback of the other two);
//   tiles on the tensor cores (mma.sync m16n8k16, bf16 operands): steps of many rows.  The matrices of a block
//     are small (a head's or a gate block's, 128 x 128 at the widths of real models), so the product is bound by
//     reading x and writing the result, and it is kept to warp-level instructions on tiles of 64 x 64 x 64;
//   a streaming kernel for steps of at most 16 rows: a warp takes an output column, its lanes walk K sixteen
//     bytes at a time, and the few rows of x come through the cache.
#include "common.cuh"

namespace zlm {

constexpr int BL_BM = 32;      // rows (tokens) of a tile
constexpr int BL_BN = 64;      // outputs of a tile
constexpr int BL_BK = 32;      // depth of a stage

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
block_linear_kernel(const TX* __restrict__ x, long x_stride, const TW* __restrict__ w, const float* __restrict__ bias,
                    TO* __restrict__ out, long out_stride, int T, int N, int K, int epi,
                    const float* __restrict__ gate, long gate_stride) {
    __shared__ float xs[BL_BK][BL_BM + 1];
    __shared__ float ws[BL_BK][BL_BN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z;
    const int n0 = blockIdx.x * BL_BN, t0 = blockIdx.y * BL_BM;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 4 outputs and 2 rows a thread
    const TX* xb = x + (long)b * K;
    const TW* wb = w + (long)b * N * K;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += BL_BK) {
        for (int i = threadIdx.x; i < BL_BM * BL_BK; i += 256) {
            const int r = i / BL_BK, k = i % BL_BK;
            const int t = t0 + r;
            xs[k][r] = (t < T && k0 + k < K) ? to_float(xb[(long)t * x_stride + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < BL_BN * BL_BK; i += 256) {
            const int r = i / BL_BK, k = i % BL_BK;
            const int n = n0 + r;
            ws[k][r] = (n < N && k0 + k < K) ? to_float(wb[(long)n * K + k0 + k]) : 0.f;
        }
        __syncthreads();
        const int kmax = min(BL_BK, K - k0);
        for (int k = 0; k < kmax; ++k) {
            const float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float wv = ws[k][tx * 4 + j];
                acc[0][j] = fmaf(a0, wv, acc[0][j]);
                acc[1][j] = fmaf(a1, wv, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int t = t0 + ty * 2 + r;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const long col = (long)b * N + n;
            float v = acc[r][j];
            if (bias) v += bias[col];
            if (epi == 1) v = 1.0f / (1.0f + expf(-v));
            else if (epi == 2) v = round_to<TO>(v) * (1.0f / (1.0f + expf(-gate[(long)t * gate_stride + col])));
            out[(long)t * out_stride + col] = from_float<TO>(v);
        }
    }
}

template <typename TO>
__device__ __forceinline__ void bl_store(TO* out, long out_stride, int t, long col, float v, const float* bias, int epi,
                                         const float* gate, long gate_stride) {
    if (bias) v += bias[col];
    if (epi == 1) v = 1.0f / (1.0f + expf(-v));
    else if (epi == 2) v = round_to<TO>(v) * (1.0f / (1.0f + expf(-gate[(long)t * gate_stride + col])));
    out[(long)t * out_stride + col] = from_float<TO>(v);
}

// ---------------------------------------------------------------- tensor cores
constexpr int MM_BM = 64, MM_BN = 64, MM_KC = 64, MM_PAD = 8;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// grid (ceil(N / 64), ceil(T / 64), B), 128 threads: warp w takes rows 16w..16w+15 of the tile and all 64 outputs.
// Needs K % 8 == 0, x_stride % 8 == 0 and 16-byte aligned bases (the host checks).
template <typename TO>
__global__ void __launch_bounds__(128)
block_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, long x_stride, const __nv_bfloat16* __restrict__ w,
                        const float* __restrict__ bias, TO* __restrict__ out, long out_stride, int T, int N, int K, int epi,
                        const float* __restrict__ gate, long gate_stride) {
    // operand tiles; when the products are done the same memory stages the tile's sums on their way out
    constexpr int LDS = MM_KC + MM_PAD, LDO = MM_BN + 1;
    __shared__ __align__(16) unsigned char raw[2 * MM_BM * LDS * 2];
    static_assert(sizeof(float) * MM_BM * LDO <= sizeof(raw), "the staged sums must fit the operand tiles");
    __nv_bfloat16 (*xs)[LDS] = reinterpret_cast<__nv_bfloat16 (*)[LDS]>(raw);
    __nv_bfloat16 (*wsm)[LDS] = reinterpret_cast<__nv_bfloat16 (*)[LDS]>(raw + MM_BM * LDS * 2);
    float* stage = reinterpret_cast<float*>(raw);
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z, n0 = blockIdx.x * MM_BN, t0 = blockIdx.y * MM_BM;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const __nv_bfloat16* xb = x + (long)b * K;
    const __nv_bfloat16* wb = w + (long)b * N * K;
    float acc[MM_BN / 8][4] = {};
    for (int k0 = 0; k0 < K; k0 += MM_KC) {
        for (int i = threadIdx.x; i < MM_BM * (MM_KC / 8); i += 128) {
            const int r = i / (MM_KC / 8), k = (i % (MM_KC / 8)) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t0 + r < T && k0 + k < K) v = *reinterpret_cast<const uint4*>(xb + (long)(t0 + r) * x_stride + k0 + k);
            *reinterpret_cast<uint4*>(&xs[r][k]) = v;
        }
        for (int i = threadIdx.x; i < MM_BN * (MM_KC / 8); i += 128) {
            const int r = i / (MM_KC / 8), k = (i % (MM_KC / 8)) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (n0 + r < N && k0 + k < K) v = *reinterpret_cast<const uint4*>(wb + (long)(n0 + r) * K + k0 + k);
            *reinterpret_cast<uint4*>(&wsm[r][k]) = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MM_KC; kk += 16) {
            uint32_t a[4];
            const int ar = warp * 16 + g;
            a[0] = *reinterpret_cast<const uint32_t*>(&xs[ar][kk + 2 * q]);
            a[1] = *reinterpret_cast<const uint32_t*>(&xs[ar + 8][kk + 2 * q]);
            a[2] = *reinterpret_cast<const uint32_t*>(&xs[ar][kk + 8 + 2 * q]);
            a[3] = *reinterpret_cast<const uint32_t*>(&xs[ar + 8][kk + 8 + 2 * q]);
#pragma unroll
            for (int j = 0; j < MM_BN / 8; ++j) {
                uint32_t bb[2];
                bb[0] = *reinterpret_cast<const uint32_t*>(&wsm[j * 8 + g][kk + 2 * q]);
                bb[1] = *reinterpret_cast<const uint32_t*>(&wsm[j * 8 + g][kk + 8 + 2 * q]);
                mma_bf16(acc[j], a, bb);
            }
        }
        __syncthreads();
    }
    // the sums go through shared memory so that a thread writes eight neighbours of a row at once
#pragma unroll
    for (int j = 0; j < MM_BN / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            stage[(warp * 16 + g + (i >= 2 ? 8 : 0)) * LDO + j * 8 + 2 * q + (i & 1)] = acc[j][i];
    __syncthreads();
    const bool wide = out_stride % 8 == 0 && ((long)b * N + n0) % 8 == 0 && (uintptr_t)out % 16 == 0 &&
                      (epi != 2 || (gate_stride % 4 == 0 && (uintptr_t)gate % 16 == 0));
    for (int idx = threadIdx.x; idx < MM_BM * (MM_BN / 8); idx += 128) {
        const int r = idx / (MM_BN / 8), c8 = (idx % (MM_BN / 8)) * 8;
        const int t = t0 + r;
        if (t >= T || n0 + c8 >= N) continue;
        const long col = (long)b * N + n0 + c8;
        if (wide && n0 + c8 + 8 <= N) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[e] = stage[r * LDO + c8 + e];
                if (bias) v[e] += bias[col + e];
                if (epi == 1) v[e] = 1.0f / (1.0f + expf(-v[e]));
            }
            if (epi == 2) {
                const float4 g0 = *reinterpret_cast<const float4*>(gate + (long)t * gate_stride + col);
                const float4 g1 = *reinterpret_cast<const float4*>(gate + (long)t * gate_stride + col + 4);
                const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = round_to<TO>(v[e]) * (1.0f / (1.0f + expf(-gv[e])));
            }
            TO* o = out + (long)t * out_stride + col;
            if (sizeof(TO) == 2) {
                uint4 pk;
                __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int e = 0; e < 4; ++e) ph[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                *reinterpret_cast<uint4*>(o) = pk;
            } else {
                *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        } else {
            for (int e = 0; e < 8 && n0 + c8 + e < N; ++e)
                bl_store<TO>(out, out_stride, t, col + e, stage[r * LDO + c8 + e], bias, epi, gate, gate_stride);
        }
    }
}

// ------------------------------------------------------------------ few rows
constexpr int SL_ROWS = 16, SL_WARPS = 8;

template <typename TW> struct BlVec;
template <> struct BlVec<float> { static constexpr int N = 4; };
template <> struct BlVec<__nv_bfloat16> { static constexpr int N = 8; };
template <typename TW> __device__ __forceinline__ void bl_load16(const TW* p, float (&f)[BlVec<TW>::N]);
template <> __device__ __forceinline__ void bl_load16<float>(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void bl_load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x; f[2 * i + 1] = v.y;
    }
}

// a warp per output column (b, n); T <= SL_ROWS; K a multiple of the 16-byte vector, aligned bases and strides
template <typename TX, typename TO>
__global__ void __launch_bounds__(SL_WARPS * 32)
block_linear_rows_kernel(const TX* __restrict__ x, long x_stride, const TX* __restrict__ w, const float* __restrict__ bias,
                         TO* __restrict__ out, long out_stride, int T, int B, int N, int K, int epi,
                         const float* __restrict__ gate, long gate_stride) {
    constexpr int V = BlVec<TX>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long col = (long)blockIdx.x * SL_WARPS + (threadIdx.x >> 5);
    if (col >= (long)B * N) return;
    const int b = (int)(col / N);
    const TX* wr = w + col * K;
    const TX* xb = x + (long)b * K;
    float acc[SL_ROWS] = {};
    for (int k = lane * V; k < K; k += 32 * V) {
        float wv[V];
        bl_load16<TX>(wr + k, wv);
#pragma unroll
        for (int t = 0; t < SL_ROWS; ++t) {
            if (t < T) {
                float xv[V];
                bl_load16<TX>(xb + (long)t * x_stride + k, xv);
#pragma unroll
                for (int i = 0; i < V; ++i) acc[t] = fmaf(xv[i], wv[i], acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < SL_ROWS; ++t) {
        if (t < T) {
            const float v = warp_sum(acc[t]);
            if (lane == 0) bl_store<TO>(out, out_stride, t, col, v, bias, epi, gate, gate_stride);
        }
    }
}

}  // namespace zlm

using namespace zlm;

// x: [T, B*K] rows with stride x_stride; w: [B, N, K] contiguous; bias: float [B*N] or null; out: [T, B*N] rows
// with stride out_stride; gate (epi 2): float rows with stride gate_stride.
ZLM_EXPORT int zlm_block_linear(const void* x, int x_dtype, long x_stride, const void* w, int w_dtype, const float* bias,
                                void* out, int out_dtype, long out_stride, int T, int B, int N, int K, int epi,
                                const float* gate, long gate_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (B <= 0 || N <= 0 || K <= 0 || epi < 0 || epi > 2 || (epi == 2 && !gate)) return ZLM_ERR_BAD_ARG;
    if (B > 65535 || (T + BL_BM - 1) / BL_BM > 65535) return ZLM_ERR_UNSUPPORTED;
    cudaError_t e;
    const int el = x_dtype == ZLM_F32 ? 4 : 2, vec = 16 / el;
    const bool aligned = x_dtype == w_dtype && K % vec == 0 && x_stride % vec == 0 && (uintptr_t)x % 16 == 0 &&
                         (uintptr_t)w % 16 == 0;
    if (aligned && T <= SL_ROWS) {
        const long cols = (long)B * N;
        dim3 sgrid((unsigned)((cols + SL_WARPS - 1) / SL_WARPS));
#define ZLM_BLR(TX, TO)                                                                                               \
    e = launch_pdl(block_linear_rows_kernel<TX, TO>, sgrid, dim3(SL_WARPS * 32), 0, stream, (const TX*)x, x_stride,     \
                   (const TX*)w, bias, (TO*)out, out_stride, T, B, N, K, epi, gate, gate_stride)
        if (x_dtype == ZLM_F32 && out_dtype == ZLM_F32) ZLM_BLR(float, float);
        else if (x_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_BLR(__nv_bfloat16, __nv_bfloat16);
        else if (x_dtype == ZLM_BF16 && out_dtype == ZLM_F32) ZLM_BLR(__nv_bfloat16, float);
        else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_BLR
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    if (aligned && x_dtype == ZLM_BF16 && (T + MM_BM - 1) / MM_BM <= 65535) {
        dim3 mgrid((N + MM_BN - 1) / MM_BN, (T + MM_BM - 1) / MM_BM, B);
        if (out_dtype == ZLM_BF16)
            e = launch_pdl(block_linear_mma_kernel<__nv_bfloat16>, mgrid, dim3(128), 0, stream, (const __nv_bfloat16*)x,
                           x_stride, (const __nv_bfloat16*)w, bias, (__nv_bfloat16*)out, out_stride, T, N, K, epi, gate,
                           gate_stride);
        else if (out_dtype == ZLM_F32)
            e = launch_pdl(block_linear_mma_kernel<float>, mgrid, dim3(128), 0, stream, (const __nv_bfloat16*)x, x_stride,
                           (const __nv_bfloat16*)w, bias, (float*)out, out_stride, T, N, K, epi, gate, gate_stride);
        else
            return ZLM_ERR_UNSUPPORTED;
        return e == cudaSuccess ? launch_status() : (int)e;
    }
    dim3 grid((N + BL_BN - 1) / BL_BN, (T + BL_BM - 1) / BL_BM, B);
#define ZLM_BL(TX, TW, TO)                                                                                          \
    e = launch_pdl(block_linear_kernel<TX, TW, TO>, grid, dim3(256), 0, stream, (const TX*)x, x_stride, (const TW*)w, \
                   bias, (TO*)out, out_stride, T, N, K, epi, gate, gate_stride)
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_F32 && out_dtype == ZLM_F32) ZLM_BL(float, float, float);
    else if (x_dtype == ZLM_BF16 && w_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_BL(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == ZLM_BF16 && w_dtype == ZLM_BF16 && out_dtype == ZLM_F32) ZLM_BL(__nv_bfloat16, __nv_bfloat16, float);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_BL
    return e == cudaSuccess ? launch_status() : (int)e;
}
