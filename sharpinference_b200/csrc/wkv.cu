// The WKV recurrence (time mixing with a per-token, per-channel decay) in float32 from per-request state.
//
// Per head, key channel i and value channel j, for the rows of a request in order:
//     w_t = exp(-exp(wraw_t + w0))                                   the decay, in (0, 1)
//     o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])           the bonus u reaches the current token only
//     S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
// then (sharpi_wkv_out) every head's o is divided by its root mean square, multiplied by a weight and by
// silu(gate), and rounded for the output projection.
//
// One block serves one (request, head) and walks the request's rows one after the other, so a row's result is
// the same sequence of operations whether it came in a prompt portion or alone.  Thread (part, j) owns KT key
// channels of value column j in registers; the partial sums of the parts meet in shared memory in a fixed
// order.  r, k, the decay and u k of the next row are staged in shared memory while the current row is
// computed: one barrier a row.
#include "common.cuh"

struct WkvArgs {
    const float* r;        // [T, heads * d]
    const float* k;
    const float* v;
    const float* wraw;     // [T, heads * d]: the decay before its two exponentials, without w0
    const float* w0;       // [heads * d]
    const float* u;        // [heads * d]
    const int* row_offsets;
    const int* state_slots;
    float* state;          // [slots, heads * d * d], [head][key][value]
    long long state_stride;
    float* o;              // [T, heads * d]
    int heads, d;
};

template <int KT>
__global__ void __launch_bounds__(1024) wkv_recurrence_kernel(WkvArgs a) {
    extern __shared__ float sm[];
    pdl_wait();
    const int d = a.d, head = blockIdx.x, b = blockIdx.y;
    const int parts = (d + KT - 1) / KT, dp = parts * KT;
    const int j = threadIdx.x % d, part = threadIdx.x / d;
    // shared: two buffers of (r, k, w, uk) [dp] each, two buffers of partial sums [parts][d]
    float* stage = sm;                        // [2][4][dp]
    float* red = sm + 2 * 4 * dp;             // [2][parts][d]
    const int first = a.row_offsets[b], end = a.row_offsets[b + 1];
    float* S_g = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)head * d * d;
    float S[KT];
#pragma unroll
    for (int i = 0; i < KT; ++i) {
        const int key = part * KT + i;
        S[i] = key < d ? S_g[(size_t)key * d + j] : 0.0f;
    }
    const size_t hd = (size_t)a.heads * d, col = (size_t)head * d;
    auto load = [&](int t, int buf) {
        float* s = stage + buf * 4 * dp;
        for (int i = threadIdx.x; i < dp; i += blockDim.x) {
            float rv = 0.0f, kv = 0.0f, wv = 0.0f, uv = 0.0f;
            if (i < d) {
                rv = a.r[(size_t)t * hd + col + i];
                kv = a.k[(size_t)t * hd + col + i];
                wv = expf(-expf(a.wraw[(size_t)t * hd + col + i] + a.w0[col + i]));
                uv = a.u[col + i] * kv;
            }
            s[i] = rv; s[dp + i] = kv; s[2 * dp + i] = wv; s[3 * dp + i] = uv;
        }
    };
    if (first < end) load(first, 0);
    __syncthreads();
    for (int t = first; t < end; ++t) {
        const int buf = (t - first) & 1;
        const float* s = stage + buf * 4 * dp + part * KT;
        const float vj = a.v[(size_t)t * hd + col + j];
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < KT; ++i) {
            const float kv = s[dp + i] * vj;
            acc += s[i] * (S[i] + s[3 * dp + i] * vj);
            S[i] = s[2 * dp + i] * S[i] + kv;
        }
        red[(buf * parts + part) * d + j] = acc;
        if (t + 1 < end) load(t + 1, buf ^ 1);
        __syncthreads();
        if (part == 0) {
            float total = 0.0f;
            for (int p = 0; p < parts; ++p) total += red[(buf * parts + p) * d + j];
            a.o[(size_t)t * hd + col + j] = total;
        }
    }
#pragma unroll
    for (int i = 0; i < KT; ++i) {
        const int key = part * KT + i;
        if (key < d) S_g[(size_t)key * d + j] = S[i];
    }
}

SHARPI_API int sharpi_wkv_recurrence(const float* r, const float* k, const float* v, const float* wraw,
                                     const float* w0, const float* u, const int* row_offsets, const int* state_slots,
                                     float* state, long long state_stride, float* o, int B, int heads, int d,
                                     cudaStream_t stream) {
    if (B <= 0) return SHARPI_OK;
    if (heads <= 0 || d <= 0 || d > 256) return SHARPI_BAD_ARGUMENT;
    WkvArgs a;
    a.r = r; a.k = k; a.v = v; a.wraw = wraw; a.w0 = w0; a.u = u; a.row_offsets = row_offsets;
    a.state_slots = state_slots; a.state = state; a.state_stride = state_stride; a.o = o; a.heads = heads; a.d = d;
    const dim3 grid(heads, B);
    if (d <= 128) {
        constexpr int KT = 16;
        const int parts = (d + KT - 1) / KT;
        const size_t smem = (size_t)(8 * parts * KT + 2 * parts * d) * sizeof(float);
        SHARPI_LAUNCH_PDL(wkv_recurrence_kernel<KT>, grid, d * parts, smem, stream, a);
    } else {
        constexpr int KT = 64;
        const int parts = (d + KT - 1) / KT;
        const size_t smem = (size_t)(8 * parts * KT + 2 * parts * d) * sizeof(float);
        SHARPI_LAUNCH_PDL(wkv_recurrence_kernel<KT>, grid, d * parts, smem, stream, a);
    }
    return SHARPI_OK;
}

// o / rms(o) * weight * silu(gate), one warp a (row, head)
template <typename TO>
__global__ void __launch_bounds__(256)
wkv_out_kernel(const float* o, const float* gate, const float* __restrict__ weight, TO* out, long long work, int heads,
               int d, float eps) {
    pdl_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= work) return;
    const int lane = threadIdx.x & 31;
    const int head = (int)(item % heads);
    const size_t base = (size_t)item * d;
    float ss = 0.0f;
    for (int i = lane; i < d; i += 32) ss += o[base + i] * o[base + i];
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32) {
        const float g = gate[base + i];
        out[base + i] = from_float<TO>(o[base + i] * scale * weight[(size_t)head * d + i] * (g / (1.0f + expf(-g))));
    }
}

SHARPI_API int sharpi_wkv_out(const float* o, const float* gate, const float* weight, void* out, int out_dtype, int T,
                              int heads, int d, float eps, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (heads <= 0 || d <= 0) return SHARPI_BAD_ARGUMENT;
    const long long work = (long long)T * heads;
    const unsigned blocks = (unsigned)((work + 7) / 8);
    if (out_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(wkv_out_kernel<float>, blocks, 256, 0, stream, o, gate, weight, (float*)out, work, heads, d, eps);
    else if (out_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(wkv_out_kernel<bf16>, blocks, 256, 0, stream, o, gate, weight, (bf16*)out, work, heads, d, eps);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}
