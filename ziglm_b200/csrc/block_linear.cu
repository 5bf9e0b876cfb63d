// Block-diagonal product: the columns of a row are cut into B equal parts and part b goes through a matrix of
// its own,
//   out[t, b*N + n] = epi( sum_k x[t, b*K + k] * W[b, n, k] + bias[b*N + n] ),   W: [B, N, K]
// This is one product per head of an attention layer (queries taken into the key latent, the latent result
// taken up to values) and the gates of a recurrence whose gate matrices are block-diagonal.
//   epi 0  nothing
//   epi 1  sigmoid(.)
//   epi 2  (.) * sigmoid(gate[t, b*N + n])      gate: float rows with a stride of their own
// CUDA cores, float accumulation.  Every output element is summed by one thread with k ascending, so a row's
// result depends on nothing but that row (not on the step's other rows or their number).
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
    dim3 grid((N + BL_BN - 1) / BL_BN, (T + BL_BM - 1) / BL_BM, B);
    cudaError_t e;
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
