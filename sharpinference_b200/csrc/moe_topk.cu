// Routing of a mixture of experts in which every row uses k experts.
//
//   router_topk   z = h Wr^T (float32), s = sigmoid(z); the k experts with the largest s + correction (the lowest
//                 index among equals) are chosen; each weight is scale * s (without the correction), divided by the
//                 sum of the chosen s first when `renormalize`.  One CTA per row: a row's logits are one fixed
//                 sequence of additions whatever else the step holds.
//   pair_tokens   after the (row, choice) pairs have been sorted by expert: the row each sorted pair belongs to.
//   combine       out[t] = add[t] + sum over the row's k pairs of y[pair], in the order of the choices.
//
// The reference routes on the host, one row at a time (src/SharpInference.Engine/ForwardPass.cs:2021-2098); here
// routing stays on the device so that a step's rows can be sorted by expert for grouped products.
#include "common.cuh"

constexpr int TOPK_WARPS = 8;

// One CTA per row: warp w forms the logits of experts w, w + 8, ... (a lane adds its elements of the row in
// ascending order in four interleaved chains, the chains and then the lanes are added in a fixed order), then
// warp 0 picks the k best.
__global__ void __launch_bounds__(TOPK_WARPS * 32)
router_topk_kernel(const float* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ correction,
                   int H, int E, int k, float scale, int renormalize, int* __restrict__ expert_id,
                   float* __restrict__ weight, float* __restrict__ scores_out) {
    extern __shared__ float smem[];                       // s [E], choice [E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    float* s_s = smem;
    float* c_s = s_s + E;
    const float* row = h + (size_t)t * H;
    for (int e = warp; e < E; e += TOPK_WARPS) {
        const float* w = wr + (size_t)e * H;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        int i = lane;
        for (; i + 96 < H; i += 128) {
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = fmaf(row[i + 32 * u], w[i + 32 * u], acc[u]);
        }
        for (int u = 0; i < H; i += 32, ++u) acc[u] = fmaf(row[i], w[i], acc[u]);
        const float z = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
        if (lane == 0) {
            const float s = 1.0f / (1.0f + expf(-z));
            s_s[e] = s;
            c_s[e] = correction ? s + correction[e] : s;
            if (scores_out) scores_out[(size_t)t * E + e] = s;
        }
    }
    __syncthreads();
    if (warp != 0) return;
    float total = 0.0f;
    int mine = 0;                                          // lane j keeps the j-th choice
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = c_s[e];
            if (c > best) { best = c; at = e; }          // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = j < E ? j : 0;                   // every score was NaN: any expert, but a valid one
        if (lane == 0) {
            expert_id[(size_t)t * k + j] = at;
            c_s[at] = -INFINITY;
        }
        if (lane == j) mine = at;
        total += s_s[at];
        __syncwarp();
    }
    const float factor = renormalize ? scale / total : scale;
    if (lane < k) weight[(size_t)t * k + lane] = s_s[mine] * factor;      // k <= 32 is checked by the host
}

SHARPI_API int sharpi_router_topk(const float* h, const float* wr, const float* correction, int T, int H, int E, int k,
                                  float scale, int renormalize, int* expert_id, float* weight, float* scores_out,
                                  cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0 || E <= 0 || k <= 0 || k > E || k > 32) return SHARPI_BAD_ARGUMENT;
    const size_t smem = (size_t)2 * E * sizeof(float);
    if (smem > 48 * 1024) return SHARPI_BAD_ARGUMENT;
    router_topk_kernel<<<T, TOPK_WARPS * 32, smem, stream>>>(h, wr, correction, H, E, k, scale, renormalize, expert_id,
                                                              weight, scores_out);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

__global__ void pair_tokens_kernel(const int* __restrict__ sorted_pairs, int P, int k, int* __restrict__ tokens) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < P) tokens[i] = sorted_pairs[i] / k;
}

SHARPI_API int sharpi_moe_pair_tokens(const int* sorted_pairs, int P, int k, int* tokens, cudaStream_t stream) {
    if (P <= 0) return SHARPI_OK;
    if (k <= 0) return SHARPI_BAD_ARGUMENT;
    pair_tokens_kernel<<<(P + 255) / 256, 256, 0, stream>>>(sorted_pairs, P, k, tokens);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* add, float* out,      // out may be add
                                   int k, int H) {
    const int t = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
        float acc = add ? add[(size_t)t * H + i] : 0.0f;
        for (int j = 0; j < k; ++j) acc += y[((size_t)t * k + j) * H + i];
        out[(size_t)t * H + i] = acc;
    }
}

SHARPI_API int sharpi_moe_combine(const float* y, const float* add, float* out, int T, int k, int H,
                                  cudaStream_t stream) {
    if (T <= 0 || H <= 0) return SHARPI_OK;
    if (k <= 0) return SHARPI_BAD_ARGUMENT;
    int by = (H + 255) / 256;
    if (by > 64) by = 64;
    moe_combine_kernel<<<dim3(T, by), 256, 0, stream>>>(y, add, out, k, H);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
