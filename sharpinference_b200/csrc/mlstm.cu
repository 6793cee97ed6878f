// The matrix-memory recurrence (mLSTM of the xLSTM family) over the rows of a step, from per-request state.
//
// Per head, with a key k_t and query q_t of size d, a value v_t of size dv, a log input gate i_t and a log forget
// gate f_t (all float32; the gates are already capped by the caller's formula below):
//
//     m_t = max(f_t + m_{t-1}, i_t)                       running maximum, m_{-1} = 0
//     a_t = exp(f_t + m_{t-1} - m_t),  b_t = exp(i_t - m_t)
//     S_t = a_t S_{t-1} + b_t k_t v_t^T                   [d, dv], S_{-1} = 0
//     n_t = a_t n_{t-1} + b_t k_t                         [d],     n_{-1} = 0
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// with i_t = cap tanh(z_i / cap), f_t = logsigmoid(cap tanh(z_f / cap)) from the raw gate projections z (bias
// added here), and q_t = q_scale * (projection).  Everything is float32: the state, the gates, every exponential
// and every product of the recurrence.  Afterwards every head's o_t is divided by its root mean square, multiplied
// by a weight and by sigmoid of an output gate.
//
// Three kernels, all reading the step through device arrays only (row_offsets, state_slots):
//   gates   one warp per (request, head) walks the request's rows in order: gates, m, a, b, n and the denominator;
//           it owns n and m of the state.  The next row's operands are loaded while this row is computed.
//   scan    one CTA per (request, head, slice of 32 value columns) walks the rows in order with its [d, 32] slice
//           of S in registers (warp w holds a band of rows, lane l column l); keys, queries and coefficients of
//           MLSTM_CHUNK rows at a time are staged in shared memory, and the bands' partial sums of S^T q meet there.
//           A row's result is one fixed sequence of operations, whatever the portion it arrived in.
//   out     one warp per (row, head): root mean square over dv, weight, output gate.
//
// State of one request and layer: per head [slices][d][32] floats of S (value columns padded with zeros to whole
// slices), then n [d], then m and three unused floats; `head_stride` floats per head.
#include "common.cuh"

constexpr int MLSTM_CHUNK = 16;      // rows staged in shared memory at a time
constexpr int MLSTM_WARPS = 8;       // warps of a scan CTA (bands of state rows)
constexpr int MLSTM_MAX_D = 256;     // key/query size the kernels take

struct MlstmArgs {
    const float* proj;       // [T, ld] fused projections of the step's rows
    int ld;
    int col_q, col_k, col_v, col_g, col_i, col_f;    // first column of each part (heads * size each)
    const float* bias_i;     // [heads]
    const float* bias_f;     // [heads]
    const int* row_offsets;  // [B + 1] first row of every request
    const int* state_slots;  // [B]
    float* state;            // [slots, state_stride]
    long long state_stride;  // floats per slot
    int head_stride;         // floats per head inside a slot
    int heads, d, dv, slices;
    float cap, q_scale;
    float* coef;             // [T, heads, 4]: a, b, denominator, unused
    float* o_raw;            // [T, heads * dv]
};

__device__ __forceinline__ float log_sigmoid(float x) {
    // -softplus(-x), formed so that neither branch overflows
    return fminf(x, 0.0f) - log1pf(expf(-fabsf(x)));
}

// ---------------------------------------------------------------------------------------
// gates: grid (B, heads), one warp
// ---------------------------------------------------------------------------------------
template <int PER_LANE>
__global__ void __launch_bounds__(32) mlstm_gates_kernel(MlstmArgs a) {
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int r0 = a.row_offsets[b], r1 = a.row_offsets[b + 1];
    if (r1 <= r0) return;
    float* st = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)h * a.head_stride;
    float* n_state = st + (size_t)a.slices * a.d * 32;
    float* m_state = n_state + a.d;
    const int d = a.d;
    float n[PER_LANE];
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        const int c = lane + 32 * j;
        n[j] = c < d ? n_state[c] : 0.0f;
    }
    float m = *m_state;
    const float bi = a.bias_i[h], bf = a.bias_f[h];

    float kq[2][PER_LANE], qq[2][PER_LANE], zi[2], zf[2];
    auto fetch = [&](int r, int buf) {
        const float* row = a.proj + (size_t)r * a.ld;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            const int c = lane + 32 * j;
            kq[buf][j] = c < d ? row[a.col_k + h * d + c] : 0.0f;
            qq[buf][j] = c < d ? row[a.col_q + h * d + c] : 0.0f;
        }
        zi[buf] = row[a.col_i + h];
        zf[buf] = row[a.col_f + h];
    };
    fetch(r0, 0);
    for (int r = r0; r < r1; ++r) {
        const int cur = (r - r0) & 1;
        if (r + 1 < r1) fetch(r + 1, cur ^ 1);
        const float ig = a.cap * tanhf((zi[cur] + bi) / a.cap);
        const float fg = log_sigmoid(a.cap * tanhf((zf[cur] + bf) / a.cap));
        const float m_new = fmaxf(fg + m, ig);
        const float ca = expf(fg + m - m_new);
        const float cb = expf(ig - m_new);
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            n[j] = fmaf(ca, n[j], cb * kq[cur][j]);
            dot = fmaf(n[j], qq[cur][j] * a.q_scale, dot);
        }
        dot = warp_sum(dot);
        m = m_new;
        if (lane == 0) {
            float* c = a.coef + ((size_t)r * a.heads + h) * 4;
            c[0] = ca;
            c[1] = cb;
            c[2] = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
        }
    }
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        const int c = lane + 32 * j;
        if (c < d) n_state[c] = n[j];
    }
    if (lane == 0) *m_state = m;
}

// ---------------------------------------------------------------------------------------
// scan: grid (B, heads, slices), MLSTM_WARPS warps; warp w holds state rows [w * BAND, (w + 1) * BAND)
// ---------------------------------------------------------------------------------------
template <int BAND>
__global__ void __launch_bounds__(MLSTM_WARPS * 32) mlstm_scan_kernel(MlstmArgs a) {
    extern __shared__ float smem[];
    const int b = blockIdx.x, h = blockIdx.y, slice = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = a.row_offsets[b], r1 = a.row_offsets[b + 1];
    if (r1 <= r0) return;
    const int d = a.d, dv = a.dv;
    constexpr int DP = BAND * MLSTM_WARPS;              // padded key size
    float* k_s = smem;                                  // [CHUNK][DP]
    float* q_s = k_s + MLSTM_CHUNK * DP;                // [CHUNK][DP]
    float* v_s = q_s + MLSTM_CHUNK * DP;                // [CHUNK][32]
    float* c_s = v_s + MLSTM_CHUNK * 32;                // [CHUNK][4]
    float* p_s = c_s + MLSTM_CHUNK * 4;                 // [CHUNK][WARPS][32]

    float* st = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)h * a.head_stride +
                (size_t)slice * d * 32;
    const int row0 = warp * BAND;
    float S[BAND];
#pragma unroll
    for (int i = 0; i < BAND; ++i) S[i] = (row0 + i < d) ? st[(size_t)(row0 + i) * 32 + lane] : 0.0f;
    const int col = slice * 32 + lane;

    for (int c0 = r0; c0 < r1; c0 += MLSTM_CHUNK) {
        const int nc = min(MLSTM_CHUNK, r1 - c0);
        __syncthreads();                                 // the previous chunk's partial sums have been read
        for (int i = threadIdx.x; i < nc * DP; i += blockDim.x) {
            const int t = i / DP, c = i - t * DP;
            const float* row = a.proj + (size_t)(c0 + t) * a.ld;
            k_s[i] = c < d ? row[a.col_k + h * d + c] : 0.0f;
            q_s[i] = c < d ? row[a.col_q + h * d + c] * a.q_scale : 0.0f;
        }
        for (int i = threadIdx.x; i < nc * 32; i += blockDim.x) {
            const int t = i >> 5, c = slice * 32 + (i & 31);
            v_s[i] = c < dv ? a.proj[(size_t)(c0 + t) * a.ld + a.col_v + h * dv + c] : 0.0f;
        }
        for (int i = threadIdx.x; i < nc * 4; i += blockDim.x)
            c_s[i] = a.coef[((size_t)(c0 + (i >> 2)) * a.heads + h) * 4 + (i & 3)];
        __syncthreads();
        for (int t = 0; t < nc; ++t) {
            const float ca = c_s[t * 4], bv = c_s[t * 4 + 1] * v_s[t * 32 + lane];
            const float* kt = k_s + t * DP + row0;
            const float* qt = q_s + t * DP + row0;
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < BAND; ++i) {
                S[i] = fmaf(ca, S[i], kt[i] * bv);
                part = fmaf(S[i], qt[i], part);
            }
            p_s[(t * MLSTM_WARPS + warp) * 32 + lane] = part;
        }
        __syncthreads();
        for (int t = warp; t < nc; t += MLSTM_WARPS) {
            float num = 0.0f;
#pragma unroll
            for (int w = 0; w < MLSTM_WARPS; ++w) num += p_s[(t * MLSTM_WARPS + w) * 32 + lane];
            if (col < dv) a.o_raw[(size_t)(c0 + t) * a.heads * dv + h * dv + col] = num / c_s[t * 4 + 2];
        }
    }
#pragma unroll
    for (int i = 0; i < BAND; ++i)
        if (row0 + i < d) st[(size_t)(row0 + i) * 32 + lane] = S[i];
}

static size_t scan_smem_bytes(int band) {
    const int dp = band * MLSTM_WARPS;
    return sizeof(float) * (size_t)(2 * MLSTM_CHUNK * dp + MLSTM_CHUNK * 32 + MLSTM_CHUNK * 4 +
                                    MLSTM_CHUNK * MLSTM_WARPS * 32);
}

template <int BAND>
static int launch_scan(const MlstmArgs& a, int B, cudaStream_t stream) {
    const size_t smem = scan_smem_bytes(BAND);
    auto kern = mlstm_scan_kernel<BAND>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SHARPI_LAUNCH_FAILED;
    kern<<<dim3(B, a.heads, a.slices), MLSTM_WARPS * 32, smem, stream>>>(a);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// The recurrence over the step's rows: leaves o_raw [T, heads * dv] (before the head norm) and the new state.
// `coef` is scratch of T * heads * 4 floats.
SHARPI_API int sharpi_mlstm_recurrence(const float* proj, int ld, int col_q, int col_k, int col_v, int col_i, int col_f,
                                       const float* bias_i, const float* bias_f, const int* row_offsets,
                                       const int* state_slots, float* state, long long state_stride, int head_stride,
                                       int B, int T, int heads, int d, int dv, float cap, float q_scale, float* coef,
                                       float* o_raw, cudaStream_t stream) {
    if (B <= 0 || T <= 0) return SHARPI_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || d > MLSTM_MAX_D || !(cap > 0.0f)) return SHARPI_BAD_ARGUMENT;
    if (heads > 65535 || (dv + 31) / 32 > 65535) return SHARPI_BAD_ARGUMENT;
    MlstmArgs a;
    a.proj = proj; a.ld = ld; a.col_q = col_q; a.col_k = col_k; a.col_v = col_v; a.col_g = 0; a.col_i = col_i;
    a.col_f = col_f; a.bias_i = bias_i; a.bias_f = bias_f; a.row_offsets = row_offsets; a.state_slots = state_slots;
    a.state = state; a.state_stride = state_stride; a.head_stride = head_stride; a.heads = heads; a.d = d; a.dv = dv;
    a.slices = (dv + 31) / 32; a.cap = cap; a.q_scale = q_scale; a.coef = coef; a.o_raw = o_raw;
    if ((long long)head_stride < (long long)a.slices * d * 32 + d + 1) return SHARPI_BAD_ARGUMENT;
    const dim3 grid(B, heads);
    if (d <= 32) mlstm_gates_kernel<1><<<grid, 32, 0, stream>>>(a);
    else if (d <= 64) mlstm_gates_kernel<2><<<grid, 32, 0, stream>>>(a);
    else if (d <= 128) mlstm_gates_kernel<4><<<grid, 32, 0, stream>>>(a);
    else mlstm_gates_kernel<8><<<grid, 32, 0, stream>>>(a);
    SHARPI_CHECK_LAUNCH();
    if (d <= 16) return launch_scan<2>(a, B, stream);
    if (d <= 32) return launch_scan<4>(a, B, stream);
    if (d <= 64) return launch_scan<8>(a, B, stream);
    if (d <= 128) return launch_scan<16>(a, B, stream);
    return launch_scan<32>(a, B, stream);
}

// ---------------------------------------------------------------------------------------
// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * w[h, :] * sigmoid(gate[t, h, :])
// One warp per (row, head).
// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void mlstm_out_kernel(const float* __restrict__ o_raw, const float* __restrict__ gate, int gate_ld,
                                 const float* __restrict__ w, float eps, long long work, int heads, int dv,
                                 TO* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= work) return;
    const long long t = item / heads;
    const int h = (int)(item - t * heads);
    const float* o = o_raw + (size_t)t * heads * dv + (size_t)h * dv;
    const float* g = gate + (size_t)t * gate_ld + (size_t)h * dv;
    float ss = 0.0f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)dv + eps);
    TO* dst = out + (size_t)t * heads * dv + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) {
        const float s = 1.0f / (1.0f + expf(-g[c]));
        dst[c] = from_float<TO>(o[c] * scale * w[h * dv + c] * s);
    }
}

SHARPI_API int sharpi_mlstm_out(const float* o_raw, const float* gate, int gate_ld, const float* w, float eps, int T,
                                int heads, int dv, void* out, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (heads <= 0 || dv <= 0) return SHARPI_BAD_ARGUMENT;
    const long long work = (long long)T * heads;
    const int warps = 8;
    const long long blocks = (work + warps - 1) / warps;
    if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32)
        mlstm_out_kernel<float><<<(unsigned)blocks, warps * 32, 0, stream>>>(o_raw, gate, gate_ld, w, eps, work, heads, dv, (float*)out);
    else if (out_dtype == SHARPI_BF16)
        mlstm_out_kernel<bf16><<<(unsigned)blocks, warps * 32, 0, stream>>>(o_raw, gate, gate_ld, w, eps, work, heads, dv, (bf16*)out);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
