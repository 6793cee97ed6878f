// The WKV recurrence (time mixing with a per-token, per-channel decay) in float32 from per-request state.
//
// Per head, key channel i and value channel j, for the rows of a request in order:
//     w_t = exp(-exp(wraw_t + w0))                                   the decay, in (0, 1)
//     o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])           the bonus u reaches the current token only
//     S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
// then (sharpi_wkv_out) every head's o is divided by its root mean square, multiplied by a weight and by
// silu(gate), and rounded for the output projection.
//
// What does not depend on the state runs first, over all rows at once (wkv_prepare_kernel): the decay with its two
// exponentials, written over wraw, and the bonus' scalar b_t = sum_i r_t[i] u[i] k_t[i], so that
// o_t[j] = sum_i r_t[i] S[i][j] + b_t v_t[j].  The walk itself (wkv_scan_kernel) is one block a (request, head): a
// thread owns a tile of S (eight key channels of four value columns) in registers; r, k, w and v of the next rows
// arrive in shared memory by cp.async, two chunks of rows on their way while a third is walked (a chunk of sixteen
// rows is walked in less time than a chunk takes to arrive).  A request's rows are walked one after the
// other and a column's parts are added in a fixed order, so a row's result is the same sequence of operations
// whether it came in a prompt portion or alone.  Heads of more than 128 elements take the form in which
// a column's key channels are dealt over several threads (wkv_recurrence_kernel).
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

__global__ void __launch_bounds__(256)
wkv_prepare_kernel(const float* r, const float* k, float* wraw, const float* __restrict__ w0,
                   const float* __restrict__ u, float* bonus, long long work, int heads, int d) {
    pdl_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= work) return;
    const int lane = threadIdx.x & 31;
    const int head = (int)(item % heads);
    const size_t base = (size_t)item * d;
    float acc = 0.0f;
    for (int i = lane; i < d; i += 32) {
        wraw[base + i] = expf(-expf(wraw[base + i] + w0[(size_t)head * d + i]));
        acc += r[base + i] * u[(size_t)head * d + i] * k[base + i];
    }
    acc = warp_sum(acc);
    if (lane == 0) bonus[item] = acc;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct WkvScanArgs {
    const float* r;        // [T, heads * d]
    const float* k;
    const float* v;
    const float* w;        // the decay itself
    const float* bonus;    // [T, heads]
    const int* row_offsets;
    const int* state_slots;
    float* state;
    long long state_stride;
    float* o;
    int heads, d, aligned;
    int ch;                // rows a chunk (at most WKV_CH; fewer when no request brings that many)
};

constexpr int WKV_CH = 16;     // rows a chunk at most
constexpr int WKV_STAGES = 3;  // chunks in shared memory: one being walked, two on their way

// Thread (kg, jg) keeps KT key channels (kg * KT ...) of CPT value columns (jg * CPT ...) of S in registers.  Per row
// it adds its part of sum_i r[i] S[i][j] into shared memory and moves its tile of S on; nothing is exchanged between
// threads inside a chunk of WKV_CH rows.  After the chunk the parts of a column are added in the order of the key
// groups, the bonus b_t v_t[j] joins, and the rows' outputs are written.
template <int KT, int CPT, int MAXT>
__global__ void __launch_bounds__(MAXT) wkv_scan_kernel(WkvScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    pdl_wait();
    const int d = a.d, head = blockIdx.x, b = blockIdx.y;
    const int KG = (d + KT - 1) / KT, DKP = KG * KT;          // key groups, keys padded
    const int JG = (d + CPT - 1) / CPT, DVP = JG * CPT;       // column groups, columns padded
    const int jg = threadIdx.x % JG, kg = threadIdx.x / JG;
    const int j0 = jg * CPT, k0 = kg * KT;
    const int CH = a.ch;
    float* stage = sm;                                        // [STAGES][CH][3][DKP]
    float* v_s = stage + WKV_STAGES * CH * 3 * DKP;           // [STAGES][CH][DVP]
    float* part = v_s + WKV_STAGES * CH * DVP;                // [CH][KG][DVP]
    float* bon = part + CH * KG * DVP;                        // [STAGES][CH]
    const int first = a.row_offsets[b], end = a.row_offsets[b + 1];
    const size_t hd = (size_t)a.heads * d, col = (size_t)head * d;
    float* S_g = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)head * d * d;
    float S[KT][CPT];
#pragma unroll
    for (int i = 0; i < KT; ++i) {
#pragma unroll
        for (int c = 0; c < CPT; ++c)
            S[i][c] = (k0 + i < d && j0 + c < d) ? S_g[(size_t)(k0 + i) * d + j0 + c] : 0.0f;
    }
    // keys and columns beyond the head's own stay zero in both buffers
    if (DKP != d)
        for (int i = threadIdx.x; i < WKV_STAGES * CH * 3 * DKP; i += blockDim.x)
            if (i % DKP >= d) stage[i] = 0.0f;
    if (DVP != d)
        for (int i = threadIdx.x; i < WKV_STAGES * CH * DVP; i += blockDim.x)
            if (i % DVP >= d) v_s[i] = 0.0f;
    auto fetch = [&](int t0, int buf) {
        const int rows = max(0, min(CH, end - t0));           // none: an empty group keeps the count of groups even
        float* st = stage + buf * CH * 3 * DKP;
        float* vs = v_s + buf * CH * DVP;
        if (a.aligned) {
            const int q = d >> 2;                              // 16-byte pieces a row and array
            for (int i = threadIdx.x; i < rows * q; i += blockDim.x) {
                const int tt = i / q, piece = (i % q) * 4;
                const size_t g = (size_t)(t0 + tt) * hd + col + piece;
                cp_async16(st + (tt * 3 + 0) * DKP + piece, a.r + g);
                cp_async16(st + (tt * 3 + 1) * DKP + piece, a.k + g);
                cp_async16(st + (tt * 3 + 2) * DKP + piece, a.w + g);
                cp_async16(vs + tt * DVP + piece, a.v + g);
            }
        } else {
            for (int i = threadIdx.x; i < rows * d; i += blockDim.x) {
                const int tt = i / d, e = i % d;
                const size_t g = (size_t)(t0 + tt) * hd + col + e;
                st[(tt * 3 + 0) * DKP + e] = a.r[g];
                st[(tt * 3 + 1) * DKP + e] = a.k[g];
                st[(tt * 3 + 2) * DKP + e] = a.w[g];
                vs[tt * DVP + e] = a.v[g];
            }
        }
        if (threadIdx.x < rows) cp_async4(bon + buf * CH + threadIdx.x, a.bonus + (size_t)(t0 + threadIdx.x) * a.heads + head);
        cp_async_commit();
    };
    fetch(first, 0);
    fetch(first + CH, 1);
    int buf = 0;
    for (int t0 = first; t0 < end; t0 += CH, buf = (buf + 1) % WKV_STAGES) {
        const int rows = min(CH, end - t0);
        cp_async_wait<1>();       // all but the newest group: this chunk is here, the next may still be on its way
        __syncthreads();          // ... for everyone; the buffer of the chunk before and the parts have been read
        fetch(t0 + 2 * CH, (buf + 2) % WKV_STAGES);          // two chunks ahead: a chunk is walked faster than one arrives
        const float* st = stage + buf * CH * 3 * DKP + k0;
        const float* vs = v_s + buf * CH * DVP + j0;
        if (kg < KG) {
#pragma unroll 2
            for (int tt = 0; tt < rows; ++tt) {
                float rk[KT], kk[KT], wk[KT], vv[CPT], acc[CPT];
#pragma unroll
                for (int i = 0; i < KT; i += 4) {
                    const float4 r4 = *reinterpret_cast<const float4*>(st + (tt * 3 + 0) * DKP + i);
                    const float4 k4 = *reinterpret_cast<const float4*>(st + (tt * 3 + 1) * DKP + i);
                    const float4 w4 = *reinterpret_cast<const float4*>(st + (tt * 3 + 2) * DKP + i);
                    rk[i] = r4.x; rk[i + 1] = r4.y; rk[i + 2] = r4.z; rk[i + 3] = r4.w;
                    kk[i] = k4.x; kk[i + 1] = k4.y; kk[i + 2] = k4.z; kk[i + 3] = k4.w;
                    wk[i] = w4.x; wk[i + 1] = w4.y; wk[i + 2] = w4.z; wk[i + 3] = w4.w;
                }
                if (CPT == 4) {
                    const float4 v4 = *reinterpret_cast<const float4*>(vs + tt * DVP);
                    vv[0] = v4.x; vv[1 % CPT] = v4.y; vv[2 % CPT] = v4.z; vv[3 % CPT] = v4.w;
                } else {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) vv[c] = vs[tt * DVP + c];
                }
#pragma unroll
                for (int c = 0; c < CPT; ++c) acc[c] = 0.0f;
#pragma unroll
                for (int i = 0; i < KT; ++i) {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        acc[c] = fmaf(rk[i], S[i][c], acc[c]);
                        S[i][c] = fmaf(wk[i], S[i][c], kk[i] * vv[c]);
                    }
                }
                if (CPT == 4) {
                    *reinterpret_cast<float4*>(part + (tt * KG + kg) * DVP + j0) =
                        make_float4(acc[0], acc[1 % CPT], acc[2 % CPT], acc[3 % CPT]);
                } else {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) part[(tt * KG + kg) * DVP + j0 + c] = acc[c];
                }
            }
        }
        __syncthreads();
        if (CPT == 4) {           // four columns a thread: d is a multiple of four and the rows of o start on 16 bytes
            for (int i = threadIdx.x; i < rows * JG; i += blockDim.x) {
                const int tt = i / JG, j = (i % JG) * 4;
                float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int g = 0; g < KG; ++g) {
                    const float4 p = *reinterpret_cast<const float4*>(part + (tt * KG + g) * DVP + j);
                    total.x += p.x; total.y += p.y; total.z += p.z; total.w += p.w;
                }
                const float bt = bon[buf * CH + tt];
                const float4 v4 = *reinterpret_cast<const float4*>(v_s + (buf * CH + tt) * DVP + j);
                *reinterpret_cast<float4*>(a.o + (size_t)(t0 + tt) * hd + col + j) =
                    make_float4(fmaf(bt, v4.x, total.x), fmaf(bt, v4.y, total.y), fmaf(bt, v4.z, total.z), fmaf(bt, v4.w, total.w));
            }
        } else {
            for (int i = threadIdx.x; i < rows * d; i += blockDim.x) {
                const int tt = i / d, j = i % d;
                float total = 0.0f;
                for (int g = 0; g < KG; ++g) total += part[(tt * KG + g) * DVP + j];
                a.o[(size_t)(t0 + tt) * hd + col + j] = fmaf(bon[buf * CH + tt], v_s[(buf * CH + tt) * DVP + j], total);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < KT; ++i) {
#pragma unroll
        for (int c = 0; c < CPT; ++c)
            if (k0 + i < d && j0 + c < d) S_g[(size_t)(k0 + i) * d + j0 + c] = S[i][c];
    }
}

template <int KT, int CPT, int MAXT>
static int launch_wkv_scan(WkvScanArgs a, int B, int T, cudaStream_t stream) {
    const int d = a.d, KG = (d + KT - 1) / KT, JG = (d + CPT - 1) / CPT;
    const int DKP = KG * KT, DVP = JG * CPT;
    const int threads = (KG * JG + 31) / 32 * 32;
    if (threads > MAXT) return SHARPI_BAD_ARGUMENT;
    a.ch = T - B + 1 < WKV_CH ? (T - B + 1 < 1 ? 1 : T - B + 1) : WKV_CH;      // no request brings more rows than T - B + 1
    const size_t per_row = (size_t)(WKV_STAGES * 3 * DKP + WKV_STAGES * DVP + WKV_STAGES + KG * DVP) * sizeof(float);
    if (a.ch * per_row > 160 * 1024) a.ch = (int)(160 * 1024 / per_row);
    if (a.ch < 1) return SHARPI_BAD_ARGUMENT;
    const size_t smem = a.ch * per_row;
    auto kern = wkv_scan_kernel<KT, CPT, MAXT>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SHARPI_LAUNCH_FAILED;
    const dim3 grid(a.heads, B);
    SHARPI_LAUNCH_PDL(kern, grid, threads, smem, stream, a);
    return SHARPI_OK;
}

SHARPI_API int sharpi_wkv_recurrence(const float* r, const float* k, const float* v, float* wraw,
                                     const float* w0, const float* u, const int* row_offsets, const int* state_slots,
                                     float* state, long long state_stride, float* o, float* bonus, int T, int B,
                                     int heads, int d, cudaStream_t stream) {
    if (B <= 0) return SHARPI_OK;
    if (heads <= 0 || d <= 0 || d > 256 || T <= 0) return SHARPI_BAD_ARGUMENT;
    if (d <= 128) {
        // the decay and the bonus' scalar for all rows at once, then the walk
        const long long work = (long long)T * heads;
        SHARPI_LAUNCH_PDL(wkv_prepare_kernel, (unsigned)((work + 7) / 8), 256, 0, stream, r, k, wraw, w0, u, bonus, work,
                          heads, d);
        WkvScanArgs s;
        s.r = r; s.k = k; s.v = v; s.w = wraw; s.bonus = bonus; s.row_offsets = row_offsets; s.state_slots = state_slots;
        s.state = state; s.state_stride = state_stride; s.o = o; s.heads = heads; s.d = d;
        const uintptr_t ptrs = reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(k) |
                               reinterpret_cast<uintptr_t>(wraw) | reinterpret_cast<uintptr_t>(v);
        s.aligned = (d % 4 == 0 && (ptrs & 15) == 0) ? 1 : 0;
        if (d % 4 == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) return launch_wkv_scan<8, 4, 512>(s, B, T, stream);
        if (d <= 88) return launch_wkv_scan<8, 1, 1024>(s, B, T, stream);
        return launch_wkv_scan<16, 1, 1024>(s, B, T, stream);
    }
    WkvArgs a;
    a.r = r; a.k = k; a.v = v; a.wraw = wraw; a.w0 = w0; a.u = u; a.row_offsets = row_offsets;
    a.state_slots = state_slots; a.state = state; a.state_stride = state_stride; a.o = o; a.heads = heads; a.d = d;
    const dim3 grid(heads, B);
    {
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
