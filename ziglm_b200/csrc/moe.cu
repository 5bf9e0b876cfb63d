// Mixture of experts: routing, the grouping of (token, choice) pairs by expert, the experts' products over those
// groups, and the weighted sum of a token's expert outputs.
//
// Routing, per token, in float:
//   score_e  = sigmoid(z_e) or z_e's softmax                              (z: router logits)
//   choice_e = score_e + correction_e                                     (correction may be absent)
//   experts form n_groups equal groups of neighbours; a group's score is the sum of its group_best largest
//   choice scores; only experts of the keep_groups best groups can be chosen (the others count as -inf);
//   the `top` experts with the largest choice scores are chosen (ties: the lower index), and their weights are
//   score_e (without the correction), divided by their sum if `renormalize`.
//
// Pair p = token * top + k.  The pairs are grouped by expert into `sorted` (offsets per expert in `offs`), and
// the rows of every expert are cut into tiles of GM rows (`tile_expert`, `tile_row`; `n_tiles[0]` tiles in all).
// The two products run over those tiles: gate/up with the activation (input rows gathered by token, output
// rows in sorted order) and down (output rows scattered to the pair's own row, float).  The sum over a token's
// pairs is taken by one thread in the order of k, so nothing depends on the step's other tokens.
#include "common.cuh"

namespace zlm {

constexpr int GM = 32, GN = 64, GK = 32;

// ------------------------------------------------------------------- routing
// one warp per token; shared: choice[E], group score[n_groups]
__global__ void route_kernel(const float* __restrict__ z, const float* __restrict__ correction, int E, int top,
                             int n_groups, int keep_groups, int group_best, int softmax_scores, int renormalize,
                             int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float sm[];
    float* score = sm;                 // [E]
    float* choice = sm + E;            // [E]
    float* gscore = sm + 2 * E;        // [n_groups]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* zr = z + (long)t * E;
    float zmax = -INFINITY, zsum = 0.f;
    if (softmax_scores) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, zr[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(zr[e] - zmax);
        zsum = warp_sum(zsum);
    }
    for (int e = lane; e < E; e += 32) {
        const float s = softmax_scores ? expf(zr[e] - zmax) / zsum : 1.0f / (1.0f + expf(-zr[e]));
        score[e] = s;
        choice[e] = correction ? s + correction[e] : s;
    }
    __syncwarp();
    if (n_groups > 1 && keep_groups < n_groups) {
        const int size = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            // the sum of the group's group_best largest choice scores: take the largest that lies below the last taken
            float total = 0.f, last = INFINITY;
            int last_i = -1;
            for (int n = 0; n < group_best && n < size; ++n) {
                float best = -INFINITY;
                int best_i = -1;
                for (int i = 0; i < size; ++i) {
                    const float c = choice[g * size + i];
                    const bool below = c < last || (c == last && i > last_i);
                    if (below && (c > best || best_i < 0)) { best = c; best_i = i; }
                }
                total += best;
                last = best; last_i = best_i;
            }
            gscore[g] = total;
        }
        __syncwarp();
        for (int g = lane; g < n_groups; g += 32) {
            int ahead = 0;
            for (int o = 0; o < n_groups; ++o)
                ahead += (gscore[o] > gscore[g] || (gscore[o] == gscore[g] && o < g)) ? 1 : 0;
            if (ahead >= keep_groups)
                for (int i = 0; i < size; ++i) choice[g * size + i] = -INFINITY;
        }
        __syncwarp();
    }
    float wsum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best || (c == best && e < best_e && c > -INFINITY)) { best = c; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;       // fewer finite candidates than `top`: cannot happen with a checked configuration
        if (lane == 0) {
            ids[(long)t * top + k] = best_e;
            weights[(long)t * top + k] = score[best_e];
            choice[best_e] = -INFINITY;
        }
        wsum += score[best_e];
        __syncwarp();
    }
    if (renormalize && lane == 0)
        for (int k = 0; k < top; ++k) weights[(long)t * top + k] /= wsum;
}

// ------------------------------------------------------------------ grouping
// one block.  counts -> offsets -> sorted pairs and tiles.
__global__ void group_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ offs, int* __restrict__ sorted,
                             int* __restrict__ tile_expert, int* __restrict__ tile_row, int* __restrict__ n_tiles) {
    extern __shared__ int smi[];
    int* count = smi;             // [E]
    int* start = smi + E;         // [E + 1]
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            offs[e] = at;
            for (int r = 0; r < count[e]; r += GM) { tile_expert[tiles] = e; tile_row[tiles] = at + r; ++tiles; }
            at += count[e];
        }
        start[E] = at;
        offs[E] = at;
        n_tiles[0] = tiles;
    }
    __syncthreads();
    // pair p goes to the place its rank among its expert's pairs gives it: pairs in ascending order
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    if (P <= 4096) {
        // few pairs: a stable order, so that a row's place does not depend on the timing of the threads
        if (threadIdx.x < E) {
            int at = start[threadIdx.x];
            for (int p = 0; p < P; ++p)
                if (ids[p] == (int)threadIdx.x) sorted[at++] = p;
        }
        for (int e = blockDim.x + threadIdx.x; e < E; e += blockDim.x) {
            int at = start[e];
            for (int p = 0; p < P; ++p)
                if (ids[p] == e) sorted[at++] = p;
        }
    } else {
        for (int p = threadIdx.x; p < P; p += blockDim.x) {
            const int e = ids[p];
            sorted[start[e] + atomicAdd(&count[e], 1)] = p;
        }
    }
}

// ----------------------------------------------------------- grouped products
// GLU: w is [E, 2N, K] (gate rows, then up rows); out[row, n] = silu(g) * u in the storage type, rows in sorted
//      order; the input row of sorted row s is token sorted[s] / top.
// else w is [E, N, K]; out[pair, n] = float, the input row is the sorted row itself.
template <typename TX, typename TW, bool GLU>
__global__ void __launch_bounds__(256)
grouped_kernel(const TX* __restrict__ x, long x_stride, const TW* __restrict__ w, void* __restrict__ out_, long out_stride,
               int N, int K, int top, const int* __restrict__ offs, const int* __restrict__ sorted,
               const int* __restrict__ tile_expert, const int* __restrict__ tile_row, const int* __restrict__ n_tiles) {
    __shared__ float xs[GK][GM + 1];
    __shared__ float ws[GLU ? 2 : 1][GK][GN + 1];
    __shared__ int row_in[GM], row_out[GM];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    if (tile >= n_tiles[0]) return;
    const int e = tile_expert[tile], r0 = tile_row[tile];
    const int rows = min(GM, offs[e + 1] - r0);
    const int n0 = blockIdx.x * GN;
    if (threadIdx.x < GM) {
        const int s = r0 + threadIdx.x;
        const int pair = threadIdx.x < rows ? sorted[s] : 0;
        row_in[threadIdx.x] = GLU ? pair / top : s;
        row_out[threadIdx.x] = GLU ? s : pair;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const TW* we = w + (long)e * (GLU ? 2 : 1) * N * K;
    float acc[GLU ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int i = threadIdx.x; i < GM * GK; i += 256) {
            const int r = i / GK, k = i % GK;
            xs[k][r] = (r < rows && k0 + k < K) ? to_float(x[(long)row_in[r] * x_stride + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < GN * GK; i += 256) {
            const int r = i / GK, k = i % GK;
            const int n = n0 + r;
            const bool ok = n < N && k0 + k < K;
            ws[0][k][r] = ok ? to_float(we[(long)n * K + k0 + k]) : 0.f;
            if (GLU) ws[1][k][r] = ok ? to_float(we[(long)(N + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
        const int kmax = min(GK, K - k0);
        for (int k = 0; k < kmax; ++k) {
            const float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1];
#pragma unroll
            for (int m = 0; m < (GLU ? 2 : 1); ++m)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float wv = ws[m][k][tx * 4 + j];
                    acc[m][0][j] = fmaf(a0, wv, acc[m][0][j]);
                    acc[m][1][j] = fmaf(a1, wv, acc[m][1][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int lr = ty * 2 + r;
        if (lr >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GLU) {
                const float g = round_to<TX>(acc[0][r][j]), u = round_to<TX>(acc[GLU ? 1 : 0][r][j]);
                ((TX*)out_)[(long)row_out[lr] * out_stride + n] = from_float<TX>((g / (1.0f + expf(-g))) * u);
            } else {
                ((float*)out_)[(long)row_out[lr] * out_stride + n] = acc[0][r][j];
            }
        }
    }
}

// out[t, :] (+)= sum_k weights[t, k] * y[t * top + k, :]
__global__ void combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, float* __restrict__ out,
                               long total, int d, int top, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / d;
    const int i = (int)(idx % d);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weights[t * top + k], y[(t * top + k) * d + i], acc);
    out[idx] = accumulate ? out[idx] + acc : acc;
}

}  // namespace zlm

using namespace zlm;

ZLM_EXPORT int zlm_moe_route(const float* z, const float* correction, int T, int E, int top, int n_groups,
                             int keep_groups, int group_best, int softmax_scores, int renormalize, int* ids,
                             float* weights, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || n_groups <= 0 || E % n_groups || keep_groups <= 0 || keep_groups > n_groups ||
        group_best <= 0 || top > keep_groups * (E / n_groups))
        return ZLM_ERR_BAD_ARG;
    const size_t smem = (2 * (size_t)E + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return ZLM_ERR_UNSUPPORTED;
    cudaError_t e = launch_pdl(route_kernel, dim3(T), dim3(32), smem, stream, z, correction, E, top, n_groups,
                               keep_groups, group_best, softmax_scores, renormalize, ids, weights);
    return e == cudaSuccess ? launch_status() : (int)e;
}

// The most tiles P pairs over E experts can make.
ZLM_EXPORT long zlm_moe_max_tiles_scratch(int P, int E) { return (long)(P + GM - 1) / GM + E; }

ZLM_EXPORT int zlm_moe_group(const int* ids, int P, int E, int* offs, int* sorted, int* tile_expert, int* tile_row,
                             int* n_tiles, cudaStream_t stream) {
    if (P <= 0) return 0;
    if (E <= 0) return ZLM_ERR_BAD_ARG;
    const size_t smem = (2 * (size_t)E + 1) * sizeof(int);
    if (smem > 48 * 1024) return ZLM_ERR_UNSUPPORTED;
    cudaError_t e = launch_pdl(group_kernel, dim3(1), dim3(1024), smem, stream, ids, P, E, offs, sorted, tile_expert,
                               tile_row, n_tiles);
    return e == cudaSuccess ? launch_status() : (int)e;
}

// glu != 0: x [T, K] (rows by token) -> out [P, N] storage type, sorted order, w [E, 2N, K]
// glu == 0: x [P, K] (sorted order)  -> out [P, N] float, pair order, w [E, N, K]
ZLM_EXPORT int zlm_moe_grouped(const void* x, int x_dtype, long x_stride, const void* w, int w_dtype, void* out,
                               long out_stride, int glu, int P, int E, int N, int K, int top, const int* offs,
                               const int* sorted, const int* tile_expert, const int* tile_row, const int* n_tiles,
                               cudaStream_t stream) {
    if (P <= 0) return 0;
    if (E <= 0 || N <= 0 || K <= 0 || top <= 0) return ZLM_ERR_BAD_ARG;
    const long max_tiles = zlm_moe_max_tiles_scratch(P, E);
    if (max_tiles > 65535) return ZLM_ERR_UNSUPPORTED;
    dim3 grid((N + GN - 1) / GN, (unsigned)max_tiles);
    cudaError_t e;
#define ZLM_GR(TX, TW, GLU)                                                                                         \
    e = launch_pdl(grouped_kernel<TX, TW, GLU>, grid, dim3(256), 0, stream, (const TX*)x, x_stride, (const TW*)w, out, \
                   out_stride, N, K, top, offs, sorted, tile_expert, tile_row, n_tiles)
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_F32) { if (glu) ZLM_GR(float, float, true); else ZLM_GR(float, float, false); }
    else if (x_dtype == ZLM_BF16 && w_dtype == ZLM_BF16) { if (glu) ZLM_GR(__nv_bfloat16, __nv_bfloat16, true); else ZLM_GR(__nv_bfloat16, __nv_bfloat16, false); }
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_GR
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_moe_combine(const float* y, const float* weights, float* out, int T, int d, int top, int accumulate,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || top <= 0) return ZLM_ERR_BAD_ARG;
    const long total = (long)T * d;
    cudaError_t e = launch_pdl(combine_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, y, weights, out,
                               total, d, top, accumulate);
    return e == cudaSuccess ? launch_status() : (int)e;
}
