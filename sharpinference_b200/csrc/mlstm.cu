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
//   gates   one warp per (request, head) walks the request's rows in order, 32 at a time: lane j holds the capped
//           gates of row j (tanh, logsigmoid; formed here, or for steps of many rows by a kernel over all rows at
//           once ahead of the walk), then every lane runs the same 32 steps of m_t = max(f_t + m_{t-1}, i_t) on
//           values passed along by shuffles (one addition and one maximum a row on the serial path), and lane j
//           leaves log a_t, log b_t and m_t of its row.  It owns m of the state.
//   scan    one CTA of 128 threads per (request, head, slice of 32 value columns) walks the rows in order with its
//           [d, 32] slice of S in registers: a thread holds d / 16 rows of four neighbouring columns, so that every
//           key and query element it reads from shared memory serves four columns.  The normaliser n is one more
//           slice whose "value" is 1 in its first column and 0 elsewhere, so n . q comes out of the same code as
//           S^T q and no CTA reads what another writes.  Keys, queries and coefficients of a chunk of rows at a time
//           are staged in shared memory (the next chunk's are on their way in registers meanwhile), and the 16
//           partial sums of every (row, column) meet there.  A row's result is one fixed sequence of operations,
//           whatever the portion it arrived in.
//   out     one warp per (row, head): the division by max(|n . q|, exp(-m)) + 1e-6, then root mean square over dv,
//           weight, output gate.
//
// State of one request and layer, per head: for every slice of 32 value columns [d][32] floats of S (columns beyond
// dv are zeros), then n [d], then m and three unused floats.  `head_stride` floats per head.
#include "common.cuh"

constexpr int MLSTM_CHUNK = 8;       // rows staged in shared memory at a time (half as many at the largest key size)
constexpr int MLSTM_MAX_D = 512;     // key/query size the kernels take

struct MlstmArgs {
    const float* proj;       // [T, ld] fused projections of the step's rows
    int ld;
    int col_q, col_k, col_v, col_i, col_f;    // first column of each part (heads * size each)
    const float* bias_i;     // [heads]
    const float* bias_f;     // [heads]
    const int* row_offsets;  // [B + 1] first row of every request
    const int* state_slots;  // [B]
    float* state;            // [slots, state_stride]
    long long state_stride;  // floats per slot
    int head_stride;         // floats per head inside a slot
    int heads, d, dv, slices;
    float cap, q_scale;
    float* coef;             // [T, heads, 4]: log a, log b, m, unused
    float* o_raw;            // [T, heads * dv]: S^T q, not yet divided
    float* nq;               // [T, heads]: n . q
};

__device__ __forceinline__ float log_sigmoid(float x) {
    // -softplus(-x), formed so that neither branch overflows
    return fminf(x, 0.0f) - log1pf(expf(-fabsf(x)));
}

// ---------------------------------------------------------------------------------------
// gates: grid (B, heads), one warp.  PRE: the capped gates of every row were formed by gate_values_kernel (all rows
// in parallel) and lie in coef[.., 0] and coef[.., 1]; otherwise the warp forms them itself (steps of few rows: one
// launch fewer).  The arithmetic is the same either way.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void capped_gates(float zi, float zf, float bi, float bf, float cap, float& ig, float& fg) {
    ig = cap * tanhf((zi + bi) / cap);
    fg = log_sigmoid(cap * tanhf((zf + bf) / cap));
}

__global__ void gate_values_kernel(MlstmArgs a, long long items) {
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= items) return;
    const long long t = item / a.heads;
    const int h = (int)(item - t * a.heads);
    float ig, fg;
    capped_gates(a.proj[(size_t)t * a.ld + a.col_i + h], a.proj[(size_t)t * a.ld + a.col_f + h], a.bias_i[h], a.bias_f[h],
                 a.cap, ig, fg);
    a.coef[item * 4] = ig;
    a.coef[item * 4 + 1] = fg;
}

template <bool PRE>
__global__ void __launch_bounds__(32) mlstm_gates_kernel(MlstmArgs a) {
    const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int r0 = a.row_offsets[b], r1 = a.row_offsets[b + 1];
    if (r1 <= r0) return;
    float* m_state = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)h * a.head_stride +
                     (size_t)a.slices * a.d * 32 + a.d;
    float m = *m_state;
    const float bi = a.bias_i[h], bf = a.bias_f[h];
    // x, y: the raw gate projections of this lane's row, or (PRE) its finished gates
    auto fetch = [&](int r, float& x, float& y) {
        x = 0.0f;
        y = 0.0f;
        if (r < r1) {
            if (PRE) {
                x = a.coef[((size_t)r * a.heads + h) * 4];
                y = a.coef[((size_t)r * a.heads + h) * 4 + 1];
            } else {
                x = a.proj[(size_t)r * a.ld + a.col_i + h];
                y = a.proj[(size_t)r * a.ld + a.col_f + h];
            }
        }
    };
    float x, y;
    fetch(r0 + lane, x, y);
    for (int t0 = r0; t0 < r1; t0 += 32) {
        const int n = min(32, r1 - t0);
        float ig = x, fg = y;
        if (!PRE) capped_gates(x, y, bi, bf, a.cap, ig, fg);
        fetch(t0 + 32 + lane, x, y);                     // the next 32 rows, while these are walked
        float m_before = 0.0f, m_after = 0.0f;
        // unrolled, so that the shuffles of all 32 rows are under way before the serial chain of additions and
        // maxima needs them; rows beyond the request's end leave m as it is
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float fj = __shfl_sync(0xffffffffu, fg, j), ij = __shfl_sync(0xffffffffu, ig, j);
            const float m_new = j < n ? fmaxf(fj + m, ij) : m;
            if (lane == j) { m_before = m; m_after = m_new; }
            m = m_new;
        }
        if (lane < n) {
            float* c = a.coef + ((size_t)(t0 + lane) * a.heads + h) * 4;
            c[0] = fg + m_before - m_after;
            c[1] = ig - m_after;
            c[2] = m_after;
        }
    }
    if (lane == 0) *m_state = m;
}

// ---------------------------------------------------------------------------------------
// scan: grid (B, heads, slices + 1), 128 threads.  Thread (warp w, group g, column group c; lane = 8 g + c) holds
// rows (4 w + g) * RT .. + RT - 1 of columns 4 c .. 4 c + 3 of its slice.
// ---------------------------------------------------------------------------------------
constexpr int SCAN_THREADS = 128;

// One float from global to shared memory without passing through a register; `take` = false writes a zero.
__device__ __forceinline__ void copy_async_f32(float* dst_shared, const float* src, bool take) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(dst_shared);
    const int bytes = take ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// CPT: value columns a thread holds (4, or 2 when the launch would otherwise leave SMs without a CTA: a CTA then
// covers 16 columns and there are twice as many).  The state's layout does not depend on it.
template <int RT, int CPT>
__global__ void __launch_bounds__(SCAN_THREADS) mlstm_scan_kernel(MlstmArgs a, int col_blocks) {
    constexpr int DP = RT * 16;                         // padded key size
    constexpr int CW = 8 * CPT;                         // value columns of a CTA
    constexpr int CHUNK = RT >= 16 ? MLSTM_CHUNK / 2 : MLSTM_CHUNK;      // rows staged at a time (48 KB of shared memory)
    constexpr int PER_THREAD = (CHUNK * DP) / SCAN_THREADS;              // staged k (and q) floats per thread
    constexpr int V_PER_THREAD = (CHUNK * CW + SCAN_THREADS - 1) / SCAN_THREADS;
    // two stages: while one chunk of rows is walked, the next one's keys, queries, values and coefficients arrive
    __shared__ __align__(16) float k_s[2][CHUNK * DP];
    __shared__ __align__(16) float q_s[2][CHUNK * DP];
    __shared__ __align__(16) float v_s[2][CHUNK * CW];
    __shared__ float c_s[2][CHUNK * 2];                 // log a, log b
    __shared__ __align__(16) float p_s[CHUNK * 16 * CW];      // [row][4 w + g][column]
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wg = warp * 4 + (lane >> 3), c4 = (lane & 7) * CPT;
    const int r0 = a.row_offsets[b], r1 = a.row_offsets[b + 1];
    if (r1 <= r0) return;
    const int d = a.d, dv = a.dv;
    const bool norm_slice = (int)blockIdx.z == col_blocks;      // the CTA that carries n in its first column
    const int col0 = blockIdx.z * CW;                   // first value column of this CTA
    float* head = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)h * a.head_stride;
    float* n_state = head + (size_t)a.slices * d * 32;
    // value column x of the head lies in slice x / 32 of the state: [slices][d][32]
    auto state_at = [&](int row, int x) -> float* { return head + ((size_t)(x >> 5) * d + row) * 32 + (x & 31); };
    const int row0 = wg * RT;
    float S[RT][CPT];
    // a thread's CPT columns are neighbours inside one slice: one 16-byte (CPT = 4) or 8-byte (CPT = 2) access a row
    // when the state's strides keep that alignment (key sizes that are multiples of four: the common case)
    const bool wide = CPT > 1 && !norm_slice && col0 + c4 + CPT <= a.slices * 32 &&
                      (reinterpret_cast<uintptr_t>(state_at(0, col0 + c4)) & (CPT * 4 - 1)) == 0;
#pragma unroll
    for (int i = 0; i < RT; ++i) {
#pragma unroll
        for (int j = 0; j < CPT; ++j) S[i][j] = 0.0f;
        if (row0 + i >= d) continue;
        if (wide) {
            const float* src = state_at(row0 + i, col0 + c4);
            if (CPT == 4) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                S[i][0] = v.x; S[i][1 % CPT] = v.y; S[i][2 % CPT] = v.z; S[i][3 % CPT] = v.w;
            } else if (CPT == 2) {
                const float2 v = *reinterpret_cast<const float2*>(src);
                S[i][0] = v.x; S[i][1 % CPT] = v.y;
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
            if (!norm_slice) { if (col0 + c4 + j < a.slices * 32) S[i][j] = *state_at(row0 + i, col0 + c4 + j); }
            else if (c4 + j == 0) S[i][j] = n_state[row0 + i];
        }
    }
    auto fetch = [&](int c0, int stage) {                // the chunk that starts at row c0, on its way into a stage
        const int nc = min(CHUNK, r1 - c0);
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int i = tid + j * SCAN_THREADS, t = i / DP, x = i - t * DP;
            const bool ok = t < nc && x < d;
            const float* row = a.proj + (size_t)(c0 + (ok ? t : 0)) * a.ld + h * d + (ok ? x : 0);
            copy_async_f32(&k_s[stage][i], row + a.col_k, ok);
            copy_async_f32(&q_s[stage][i], row + a.col_q, ok);
        }
#pragma unroll
        for (int j = 0; j < V_PER_THREAD; ++j) {
            const int i = tid + j * SCAN_THREADS, t = i / CW, x = i - t * CW;
            if (i < CHUNK * CW) {
                if (norm_slice) {
                    v_s[stage][i] = (t < nc && x == 0) ? 1.0f : 0.0f;
                } else {
                    const bool ok = t < nc && col0 + x < dv;
                    copy_async_f32(&v_s[stage][i], a.proj + (size_t)(c0 + (ok ? t : 0)) * a.ld + a.col_v + h * dv +
                                                       (ok ? col0 + x : 0), ok);
                }
            }
        }
        if (tid < CHUNK * 2) {
            const bool ok = (tid >> 1) < nc;
            copy_async_f32(&c_s[stage][tid], a.coef + ((size_t)(c0 + (ok ? tid >> 1 : 0)) * a.heads + h) * 4 + (tid & 1), ok);
        }
        copy_async_commit();
    };
    fetch(r0, 0);
    int stage = 0;
    for (int c0 = r0; c0 < r1; c0 += CHUNK, stage ^= 1) {
        const int nc = min(CHUNK, r1 - c0);
        copy_async_wait_all();
        __syncthreads();              // this chunk has arrived; the other stage and the partial sums have been read
        if (c0 + CHUNK < r1) fetch(c0 + CHUNK, stage ^ 1);
        float ea[CHUNK], eb[CHUNK];                      // a_t and b_t of the chunk, ahead of the serial walk
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) {
            ea[t] = expf(c_s[stage][t * 2]);
            eb[t] = expf(c_s[stage][t * 2 + 1]);
        }
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) {
            if (t >= nc) break;
            const float ca = ea[t], cb = eb[t];
            float bv[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) bv[j] = cb * v_s[stage][t * CW + c4 + j];
            const float* kt = &k_s[stage][t * DP + row0];
            const float* qt = &q_s[stage][t * DP + row0];
            float part[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) part[j] = 0.0f;
#pragma unroll
            for (int i = 0; i < RT; ++i) {
                const float kk = kt[i], qq = qt[i];
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    S[i][j] = fmaf(ca, S[i][j], kk * bv[j]);
                    part[j] = fmaf(S[i][j], qq, part[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < CPT; ++j) p_s[(t * 16 + wg) * CW + c4 + j] = part[j];
        }
        __syncthreads();
        for (int idx = tid; idx < nc * CW; idx += SCAN_THREADS) {
            const int t = idx / CW, x = idx - t * CW;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < 16; ++w) sum += p_s[(t * 16 + w) * CW + x];
            sum *= a.q_scale;                            // the query's factor, applied to the finished sum
            if (norm_slice) {
                if (x == 0) a.nq[(size_t)(c0 + t) * a.heads + h] = sum;
            } else if (col0 + x < dv) {
                a.o_raw[(size_t)(c0 + t) * a.heads * dv + h * dv + col0 + x] = sum;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < RT; ++i) {
        if (row0 + i >= d) continue;
        if (wide) {
            float* dst = state_at(row0 + i, col0 + c4);
            if (CPT == 4) *reinterpret_cast<float4*>(dst) = make_float4(S[i][0], S[i][1 % CPT], S[i][2 % CPT], S[i][3 % CPT]);
            else if (CPT == 2) *reinterpret_cast<float2*>(dst) = make_float2(S[i][0], S[i][1 % CPT]);
            continue;
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
            if (!norm_slice) { if (col0 + c4 + j < a.slices * 32) *state_at(row0 + i, col0 + c4 + j) = S[i][j]; }
            else if (c4 + j == 0) n_state[row0 + i] = S[i][j];
        }
    }
}

template <int RT>
static int launch_scan(const MlstmArgs& a, int B, cudaStream_t stream) {
    // CTAs of 32 columns unless they would be fewer than the SMs (a single prompt portion): then of 16.  (CTAs of 8
    // columns, twice as many again, measured slower: 488 against 390 us for one portion of 2048 rows, 8 heads.)
    if ((long long)B * a.heads * (a.slices + 1) >= 148) {
        mlstm_scan_kernel<RT, 4><<<dim3(B, a.heads, a.slices + 1), SCAN_THREADS, 0, stream>>>(a, a.slices);
    } else {
        const int blocks = (a.dv + 15) / 16;
        mlstm_scan_kernel<RT, 2><<<dim3(B, a.heads, blocks + 1), SCAN_THREADS, 0, stream>>>(a, blocks);
    }
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// The recurrence over the step's rows: leaves the numerators o_raw [T, heads * dv], n . q in nq [T, heads], the
// running maximum of every row in coef[.., 2] (coef: T * heads * 4 floats) and the new state.
SHARPI_API int sharpi_mlstm_recurrence(const float* proj, int ld, int col_q, int col_k, int col_v, int col_i, int col_f,
                                       const float* bias_i, const float* bias_f, const int* row_offsets,
                                       const int* state_slots, float* state, long long state_stride, int head_stride,
                                       int B, int T, int heads, int d, int dv, float cap, float q_scale, float* coef,
                                       float* o_raw, float* nq, cudaStream_t stream) {
    if (B <= 0 || T <= 0) return SHARPI_OK;
    if (heads <= 0 || d <= 0 || dv <= 0 || d > MLSTM_MAX_D || !(cap > 0.0f)) return SHARPI_BAD_ARGUMENT;
    if (heads > 65535 || (dv + 31) / 32 + 1 > 65535) return SHARPI_BAD_ARGUMENT;
    MlstmArgs a;
    a.proj = proj; a.ld = ld; a.col_q = col_q; a.col_k = col_k; a.col_v = col_v; a.col_i = col_i;
    a.col_f = col_f; a.bias_i = bias_i; a.bias_f = bias_f; a.row_offsets = row_offsets; a.state_slots = state_slots;
    a.state = state; a.state_stride = state_stride; a.head_stride = head_stride; a.heads = heads; a.d = d; a.dv = dv;
    a.slices = (dv + 31) / 32; a.cap = cap; a.q_scale = q_scale; a.coef = coef; a.o_raw = o_raw; a.nq = nq;
    if ((long long)head_stride < (long long)a.slices * d * 32 + d + 1) return SHARPI_BAD_ARGUMENT;
    if (T > 256) {                   // many rows: the gates' tanh and logsigmoid for all rows at once, ahead of the walk
        const long long items = (long long)T * heads;
        gate_values_kernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(a, items);
        SHARPI_CHECK_LAUNCH();
        mlstm_gates_kernel<true><<<dim3(B, heads), 32, 0, stream>>>(a);
    } else {
        mlstm_gates_kernel<false><<<dim3(B, heads), 32, 0, stream>>>(a);
    }
    SHARPI_CHECK_LAUNCH();
    if (d <= 16) return launch_scan<1>(a, B, stream);
    if (d <= 32) return launch_scan<2>(a, B, stream);
    if (d <= 64) return launch_scan<4>(a, B, stream);
    if (d <= 128) return launch_scan<8>(a, B, stream);
    if (d <= 256) return launch_scan<16>(a, B, stream);
    return launch_scan<32>(a, B, stream);
}

// ---------------------------------------------------------------------------------------
// o[t, h, :] = num[t, h, :] / (max(|nq[t, h]|, exp(-m[t, h])) + 1e-6)
// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * w[h, :] * sigmoid(gate[t, h, :])
// One warp per (row, head).
// ---------------------------------------------------------------------------------------
constexpr int OUT_REGS = 8;      // value sizes up to 32 * OUT_REGS are held in registers by the out kernel

template <typename TO>
__global__ void mlstm_out_kernel(const float* __restrict__ o_raw, const float* __restrict__ nq,
                                 const float* __restrict__ coef, const float* __restrict__ gate, int gate_ld,
                                 const float* __restrict__ w, float eps, long long work, int heads, int dv,
                                 TO* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= work) return;
    const long long t = item / heads;
    const int h = (int)(item - t * heads);
    const float* o = o_raw + (size_t)t * heads * dv + (size_t)h * dv;
    const float* g = gate + (size_t)t * gate_ld + (size_t)h * dv;
    const float den = fmaxf(fabsf(nq[item]), expf(-coef[item * 4 + 2])) + 1e-6f;
    TO* dst = out + (size_t)t * heads * dv + (size_t)h * dv;
    if (dv <= 32 * OUT_REGS) {
        // the head's values and gates in registers: every load is under way before the first is used
        float v[OUT_REGS], gg[OUT_REGS], ww[OUT_REGS];
#pragma unroll
        for (int r = 0; r < OUT_REGS; ++r) {
            const int c = lane + 32 * r;
            v[r] = c < dv ? o[c] : 0.0f;
            gg[r] = c < dv ? g[c] : 0.0f;
            ww[r] = c < dv ? w[h * dv + c] : 0.0f;
        }
        float ss = 0.0f;
#pragma unroll
        for (int r = 0; r < OUT_REGS; ++r) {
            v[r] = v[r] / den;
            ss = fmaf(v[r], v[r], ss);
        }
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)dv + eps);
#pragma unroll
        for (int r = 0; r < OUT_REGS; ++r) {
            const int c = lane + 32 * r;
            if (c < dv) dst[c] = from_float<TO>(v[r] * scale * ww[r] * (1.0f / (1.0f + expf(-gg[r]))));
        }
        return;
    }
    float ss = 0.0f;
    for (int c = lane; c < dv; c += 32) {
        const float v = o[c] / den;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        const float s = 1.0f / (1.0f + expf(-g[c]));
        dst[c] = from_float<TO>(o[c] / den * scale * w[h * dv + c] * s);
    }
}

SHARPI_API int sharpi_mlstm_out(const float* o_raw, const float* nq, const float* coef, const float* gate, int gate_ld, const float* w, float eps, int T,
                                int heads, int dv, void* out, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (heads <= 0 || dv <= 0) return SHARPI_BAD_ARGUMENT;
    const long long work = (long long)T * heads;
    const int warps = 8;
    const long long blocks = (work + warps - 1) / warps;
    if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32)
        mlstm_out_kernel<float><<<(unsigned)blocks, warps * 32, 0, stream>>>(o_raw, nq, coef, gate, gate_ld, w, eps, work, heads, dv, (float*)out);
    else if (out_dtype == SHARPI_BF16)
        mlstm_out_kernel<bf16><<<(unsigned)blocks, warps * 32, 0, stream>>>(o_raw, nq, coef, gate, gate_ld, w, eps, work, heads, dv, (bf16*)out);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
