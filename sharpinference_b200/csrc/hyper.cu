// Several residual streams per token (hyper-connections), the token shift, and the embedding with a hashed
// pair table.  Everything here is float32 arithmetic; a block serves one row of the step (one group of a row in the
// grouped norm, a tile of a row's columns in the token shift) with a block size that the width alone decides, so a
// row's result is the same sequence of operations whatever else is in the batch.
//
//   sharpi_embed_pair      x = embed[token] + pair[(prev * mul_prev + token * mul_cur) mod buckets], the row
//                          `buckets` for a sequence's first token; written to every stream.  The previous
//                          token of a request is per-request state (stored as token + 1, so that a zeroed
//                          slot means "none").
//   sharpi_hc_mix_norm     with S streams x_1..x_S per row and a sublayer output y not yet added:
//                          x_t <- sum_s mix[s, t] x_s + out[t] y (all t from the old x), then
//                          u = sum_t in[t] x_t (or the plain sum), and u normed in G consecutive groups,
//                          each by its own sqrt(mean(u^2) + eps), times a weight.  The update of the streams
//                          is fused into the norm that reads them next, the way a residual add is.
//   sharpi_token_shift     out_k = h + (h' - h) * mu_k for K vectors mu_k, h' the previous row of the same
//                          request, or the request's stored row for the first row of a portion; the stored
//                          row becomes the portion's last h.
//   sharpi_norm_mean2      scale * (rms(a) * wa + rms(b) * wb) row by row: two branches of a mixer joined.
#include "common.cuh"

constexpr int HC_MAX_STREAMS = 8;

template <typename TT>
__global__ void __launch_bounds__(1024)
embed_pair_kernel(const int* ids, const TT* __restrict__ embed, const TT* __restrict__ pairs, const int* row_request,
                  const int* row_offsets, const int* state_slots, int* prev_state, float* out, int H, int S, int V,
                  int buckets, int mul_prev, int mul_cur) {
    pdl_wait();
    __shared__ int s_prev;
    const int t = blockIdx.x;
    const int b = row_request[t];
    const int first = row_offsets[b];
    if (threadIdx.x == 0) {
        if (t == first) {
            const int slot = state_slots[b];
            s_prev = prev_state[slot] - 1;
            prev_state[slot] = ids[row_offsets[b + 1] - 1] + 1;     // only this block touches the request's word
        } else {
            s_prev = ids[t - 1];
        }
    }
    __syncthreads();
    int tok = ids[t];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    long long row = buckets;
    if (s_prev >= 0) {
        row = ((long long)s_prev * mul_prev + (long long)tok * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const TT* e = embed + (size_t)tok * H;
    const TT* p = pairs + (size_t)row * H;
    float* o = out + (size_t)t * S * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = to_float(e[c]) + to_float(p[c]);
        for (int s = 0; s < S; ++s) o[(size_t)s * H + c] = v;
    }
}

SHARPI_API int sharpi_embed_pair(const int* ids, const void* embed, const void* pairs, int table_dtype,
                                 const int* row_request, const int* row_offsets, const int* state_slots,
                                 int* prev_state, float* out, int T, int H, int S, int V, int buckets, int mul_prev,
                                 int mul_cur, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0 || S <= 0 || V <= 0 || buckets <= 0) return SHARPI_BAD_ARGUMENT;
    const int threads = H >= 1024 ? 1024 : (H + 31) / 32 * 32;
    if (table_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(embed_pair_kernel<float>, T, threads, 0, stream, ids, (const float*)embed, (const float*)pairs,
                          row_request, row_offsets, state_slots, prev_state, out, H, S, V, buckets, mul_prev, mul_cur);
    else if (table_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(embed_pair_kernel<bf16>, T, threads, 0, stream, ids, (const bf16*)embed, (const bf16*)pairs,
                          row_request, row_offsets, state_slots, prev_state, out, H, S, V, buckets, mul_prev, mul_cur);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}

struct HcArgs {
    float* x;            // [T, S, H]
    const float* y;      // [T, H] or null: nothing pending
    const float* mix;    // [S, S] indexed [from, to]
    const float* outc;   // [S]
    const float* inc;    // [S] or null: the plain sum of the streams
    const float* w;      // [H]
    const int* rows;     // gather: only these rows, x is left as it is
    void* h;             // [R, H]
    int H, S, G;
    float eps;
};

// PER_GROUP: a block serves one group of one row (small steps: more blocks, one pass); otherwise a block serves a
// row, group after group.  The block size and the order of every sum are the same either way, so a row's result
// does not depend on which form ran.
template <typename TO, bool PER_GROUP>
__global__ void __launch_bounds__(256) hc_mix_norm_kernel(HcArgs a) {
    extern __shared__ float u_sm[];              // the group's columns of u
    __shared__ float red[32];
    __shared__ float coef[HC_MAX_STREAMS * HC_MAX_STREAMS + 2 * HC_MAX_STREAMS];
    pdl_wait();
    const int S = a.S, H = a.H;
    float* mix = coef;
    float* outc = coef + HC_MAX_STREAMS * HC_MAX_STREAMS;
    float* inc = outc + HC_MAX_STREAMS;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix[i] = a.y ? a.mix[i] : 0.0f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        outc[i] = a.y ? a.outc[i] : 0.0f;
        inc[i] = a.inc ? a.inc[i] : 1.0f;
    }
    __syncthreads();
    // the groups are normed apart, so nothing passes between blocks
    const int r = blockIdx.x;
    const int row = a.rows ? a.rows[r] : r;
    const int gs = H / a.G;
    float* xr = a.x + (size_t)row * S * H;
    const int g_first = PER_GROUP ? blockIdx.y : 0, g_end = PER_GROUP ? blockIdx.y + 1 : a.G;
    for (int g = g_first; g < g_end; ++g) {
        const int c0 = g * gs;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const int c = c0 + i;
            float xs[HC_MAX_STREAMS];
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s) xs[s] = s < S ? xr[(size_t)s * H + c] : 0.0f;
            float u = 0.0f;
            if (a.y) {
                const float yv = a.y[(size_t)row * H + c];
#pragma unroll
                for (int t = 0; t < HC_MAX_STREAMS; ++t) {
                    if (t < S) {
                        float v = 0.0f;
#pragma unroll
                        for (int s = 0; s < HC_MAX_STREAMS; ++s)
                            if (s < S) v += mix[s * S + t] * xs[s];
                        v += outc[t] * yv;
                        if (!a.rows) xr[(size_t)t * H + c] = v;
                        u += inc[t] * v;
                    }
                }
            } else {
#pragma unroll
                for (int t = 0; t < HC_MAX_STREAMS; ++t)
                    if (t < S) u += inc[t] * xs[t];
            }
            u_sm[i] = u;
            ss += u * u;
        }
        const float total = block_sum(ss, red);
        const float scale = 1.0f / sqrtf(total / (float)gs + a.eps);
        TO* out = (TO*)a.h + (size_t)r * H + c0;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) out[i] = from_float<TO>(u_sm[i] * scale * a.w[c0 + i]);
        __syncthreads();          // u_sm is the next group's
    }
}

SHARPI_API int sharpi_hc_mix_norm(float* x, const float* y, const float* mix, const float* outc, const float* inc,
                                  const float* w, const int* rows, void* h, int h_dtype, int R, int H, int S, int G,
                                  float eps, cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (H <= 0 || S <= 0 || S > HC_MAX_STREAMS || G <= 0 || H % G != 0) return SHARPI_BAD_ARGUMENT;
    if ((size_t)(H / G) * sizeof(float) > 200 * 1024) return SHARPI_BAD_ARGUMENT;
    HcArgs a;
    a.x = x; a.y = y; a.mix = mix; a.outc = outc; a.inc = inc; a.w = w; a.rows = rows; a.h = h;
    a.H = H; a.S = S; a.G = G; a.eps = eps;
    const int gs = H / G;
    const size_t smem = (size_t)gs * sizeof(float);
    const int threads = gs >= 256 ? 256 : (gs + 31) / 32 * 32;       // the same for both forms
    const bool per_group = R <= 256;
#define HC_CASE(TO, PG)                                                                                         \
    do {                                                                                                        \
        auto kern = hc_mix_norm_kernel<TO, PG>;                                                                 \
        if (smem > 48 * 1024 &&                                                                                 \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)  \
            return SHARPI_LAUNCH_FAILED;                                                                        \
        SHARPI_LAUNCH_PDL(kern, dim3(R, PG ? G : 1), threads, smem, stream, a);                                 \
    } while (0)
    if (h_dtype == SHARPI_F32) { if (per_group) HC_CASE(float, true); else HC_CASE(float, false); }
    else if (h_dtype == SHARPI_BF16) { if (per_group) HC_CASE(bf16, true); else HC_CASE(bf16, false); }
    else return SHARPI_BAD_ARGUMENT;
#undef HC_CASE
    return SHARPI_OK;
}

// CPT columns a thread: one in small steps (more blocks), four in large ones (all loads of a thread in flight
// before its first store).  Element by element the arithmetic is the same.
template <typename TO, int CPT>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* h, const float* __restrict__ mu, float* state, long long state_stride,
                   const int* row_request, const int* row_offsets, const int* state_slots, TO* out, int T, int H,
                   int K) {
    pdl_wait();
    const int t = blockIdx.x;
    const int base = blockIdx.y * blockDim.x * CPT + threadIdx.x;
    const int b = row_request[t];
    const int first = row_offsets[b];
    const bool is_first = t == first;
    float* st = state + (size_t)state_slots[b] * state_stride;
    const float* prev = is_first ? st : h + (size_t)(t - 1) * H;
    const float* last = h + (size_t)(row_offsets[b + 1] - 1) * H;
    float hv[CPT], pv[CPT], lv[CPT];
#pragma unroll
    for (int q = 0; q < CPT; ++q) {
        const int c = base + q * blockDim.x;
        hv[q] = c < H ? h[(size_t)t * H + c] : 0.0f;
        pv[q] = c < H ? prev[c] : 0.0f;
        lv[q] = (is_first && c < H) ? last[c] : 0.0f;
    }
#pragma unroll
    for (int q = 0; q < CPT; ++q) {
        const int c = base + q * blockDim.x;
        if (c >= H) continue;
        const float d = pv[q] - hv[q];
        for (int k = 0; k < K; ++k)
            out[((size_t)k * T + t) * H + c] = from_float<TO>(hv[q] + d * mu[(size_t)k * H + c]);
        // this thread has read st[c]; no other thread of the launch touches this element of the request's row
        if (is_first) st[c] = lv[q];
    }
}

SHARPI_API int sharpi_token_shift(const float* h, const float* mu, float* state, long long state_stride,
                                  const int* row_request, const int* row_offsets, const int* state_slots, void* out,
                                  int out_dtype, int T, int H, int K, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0 || K <= 0) return SHARPI_BAD_ARGUMENT;
    const bool wide = T >= 512;
    const dim3 grid(T, (H + (wide ? 1024 : 256) - 1) / (wide ? 1024 : 256));
#define TS_CASE(TO, CPT)                                                                                       \
    SHARPI_LAUNCH_PDL((token_shift_kernel<TO, CPT>), grid, 256, 0, stream, h, mu, state, state_stride, row_request, \
                      row_offsets, state_slots, (TO*)out, T, H, K)
    if (out_dtype == SHARPI_F32) { if (wide) TS_CASE(float, 4); else TS_CASE(float, 1); }
    else if (out_dtype == SHARPI_BF16) { if (wide) TS_CASE(bf16, 4); else TS_CASE(bf16, 1); }
    else return SHARPI_BAD_ARGUMENT;
#undef TS_CASE
    return SHARPI_OK;
}

__global__ void __launch_bounds__(1024)
norm_mean2_kernel(const float* a, const float* __restrict__ wa, const float* b, const float* __restrict__ wb,
                  float* out, int H, float eps, float scale) {
    __shared__ float red[32];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float av = a[base + c], bv = b[base + c];
        sa += av * av;
        sb += bv * bv;
    }
    sa = block_sum(sa, red);
    sb = block_sum(sb, red);
    const float ra = 1.0f / sqrtf(sa / (float)H + eps), rb = 1.0f / sqrtf(sb / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[base + c] = scale * (a[base + c] * ra * wa[c] + b[base + c] * rb * wb[c]);
}

SHARPI_API int sharpi_norm_mean2(const float* a, const float* wa, const float* b, const float* wb, float* out, int T,
                                 int H, float eps, float scale, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0) return SHARPI_BAD_ARGUMENT;
    const int threads = H >= 1024 ? 1024 : (H + 31) / 32 * 32;
    SHARPI_LAUNCH_PDL(norm_mean2_kernel, T, threads, 0, stream, a, wa, b, wb, out, H, eps, scale);
    return SHARPI_OK;
}
