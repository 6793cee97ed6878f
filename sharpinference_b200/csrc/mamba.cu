// The selective state-space scan (Mamba) from per-request state, and the short causal convolution before it.
//
//   sharpi_causal_conv   (optionally the silu of a second block of columns, the scan's gate, in place, and)
//                        x_t[c] = silu(b[c] + sum_j w[c][j] in_{t - (taps - 1 - j)}[c]): the last column of w is
//                        the current token's.  Inputs before a portion's first row come from the request's state
//                        (its last taps - 1 inputs; zeros at a sequence's start), which a second launch then
//                        moves on to the portion's last inputs.
//   sharpi_slice_cols    a block of columns of a float32 matrix as a contiguous matrix in the activation dtype
//                        (the step-size inputs of the scan, cut out of the fused projection).
//   sharpi_selective_scan  per channel c and state n, for the rows of a request in order:
//                            S[c][n] <- exp(dt[c] A[c][n]) S[c][n] + dt[c] x[c] B[n],  A = -exp(A_log)
//                            y[c] = sum_n S[c][n] C[n] + D[c] x[c],  out = y g[c]
//                        with dt the step sizes (after their softplus) and g the gate (after its silu),
//                        all in float32 (exp(dt A) as exp2 of dt A log2(e)).  A group of lanes owns one channel,
//                        each lane eight states in registers; the sum over the states is a fixed tree of exchanges,
//                        and the walk over a request's rows is sequential, so a row's result does not depend on how
//                        the prompt was cut or batched.
#include "common.cuh"

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// 2^x for x <= 0 in one special-function instruction (two units in the last place; results below the smallest
// normal number become zero, which is what a decay that small is).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* in, int ld, const float* __restrict__ w, const float* __restrict__ bias,
                   const float* state, long long state_stride, const int* row_request, const int* row_offsets,
                   const int* state_slots, float* x32, TO* xact, int C, int taps, float* gate) {
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    if (gate) gate[(size_t)t * ld + c] = silu_f(gate[(size_t)t * ld + c]);
    const int b = row_request[t];
    const int i = t - row_offsets[b];                 // place within the portion
    const float* st = state + (size_t)state_slots[b] * state_stride;      // [taps - 1][C], oldest first
    float acc = bias ? bias[c] : 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float v = (i - back >= 0) ? in[(size_t)(t - back) * ld + c] : st[(size_t)(taps - 1 + i - back) * C + c];
        acc += w[(size_t)c * taps + j] * v;
    }
    const float y = silu_f(acc);
    x32[(size_t)t * C + c] = y;
    if (xact) xact[(size_t)t * C + c] = from_float<TO>(y);
}

__global__ void __launch_bounds__(256)
causal_conv_state_kernel(const float* in, int ld, float* state, long long state_stride, const int* row_offsets,
                         const int* state_slots, int C, int taps) {
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = row_offsets[b], n = row_offsets[b + 1] - first, K = taps - 1;
    float* st = state + (size_t)state_slots[b] * state_stride;
    for (int j = 0; j < K; ++j) {                      // ascending: st[j + n] is read before it is overwritten
        const int src = n - K + j;
        st[(size_t)j * C + c] = src >= 0 ? in[(size_t)(first + src) * ld + c] : st[(size_t)(j + n) * C + c];
    }
}

SHARPI_API int sharpi_causal_conv(const float* in, int ld, const float* w, const float* bias, float* state,
                                  long long state_stride, const int* row_request, const int* row_offsets,
                                  const int* state_slots, float* x32, void* xact, int act_dtype, int T, int B, int C,
                                  int taps, int gate_col, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (C <= 0 || taps <= 0 || B <= 0 || gate_col + C > ld || (gate_col >= 0 && gate_col < C)) return SHARPI_BAD_ARGUMENT;
    float* gate = gate_col >= 0 ? const_cast<float*>(in) + gate_col : nullptr;
    const dim3 grid(T, (C + 255) / 256);
    if (act_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(causal_conv_kernel<float>, grid, 256, 0, stream, in, ld, w, bias, (const float*)state,
                          state_stride, row_request, row_offsets, state_slots, x32, (float*)nullptr, C, taps, gate);
    else if (act_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(causal_conv_kernel<bf16>, grid, 256, 0, stream, in, ld, w, bias, (const float*)state,
                          state_stride, row_request, row_offsets, state_slots, x32, (bf16*)xact, C, taps, gate);
    else
        return SHARPI_BAD_ARGUMENT;
    if (taps > 1) {
        causal_conv_state_kernel<<<dim3((C + 255) / 256, B), 256, 0, stream>>>(in, ld, state, state_stride, row_offsets,
                                                                               state_slots, C, taps);
        SHARPI_CHECK_LAUNCH();
    }
    return SHARPI_OK;
}

template <typename TO>
__global__ void __launch_bounds__(256)
slice_cols_kernel(const float* src, int ld, int col0, int ncols, TO* out, long long total) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / ncols;
    const int c = (int)(i % ncols);
    out[i] = from_float<TO>(src[(size_t)t * ld + col0 + c]);
}

SHARPI_API int sharpi_slice_cols(const float* src, int ld, int col0, int ncols, void* out, int out_dtype, int T,
                                 cudaStream_t stream) {
    if (T <= 0 || ncols <= 0) return SHARPI_OK;
    if (col0 < 0 || col0 + ncols > ld) return SHARPI_BAD_ARGUMENT;
    const long long total = (long long)T * ncols;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(slice_cols_kernel<float>, blocks, 256, 0, stream, src, ld, col0, ncols, (float*)out, total);
    else if (out_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(slice_cols_kernel<bf16>, blocks, 256, 0, stream, src, ld, col0, ncols, (bf16*)out, total);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}

struct ScanArgs {
    const float* x;          // [T, C] after convolution and silu
    const float* dtraw;      // [T, C]: the step sizes (after bias and softplus)
    const float* bc;         // [T, ld_bc]: B at col_b, C at col_c, N columns each
    int ld_bc, col_b, col_c;
    const float* a_log;      // [C, N]
    const float* dskip;      // [C]
    const float* z;          // [T, ld_z]: the gate (after its silu)
    int ld_z;
    const int* row_offsets;
    const int* state_slots;
    float* state;            // [slots, C * N]
    long long state_stride;
    void* out;               // [T, C]
    int C, N;
    int vec_ch, vec_bc;      // whether the channel arrays / B and C may be fetched 16 bytes at a time
    int ch;                  // rows a chunk (at most SCAN_CH; fewer when no request brings that many)
};

constexpr int SCAN_NPT = 8;      // states a lane keeps
constexpr int SCAN_CH = 16;      // rows a chunk at most
constexpr int SCAN_STAGES = 3;   // chunks in shared memory: one being walked, two on their way

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A block of W warps (four, or one when that is what it takes to give every SM a block) serves CPB = W * 32 / G
// channels of one request.  The rows' inputs arrive in shared memory
// by cp.async, two chunks of SCAN_CH rows on their way while a third is walked: per row the block's channels of dtraw, x and z and the row's B
// and C.  What does not depend on the state (the softplus of the step sizes, the silu of the gate) was formed over
// all rows at once by the kernels before this one.
template <typename TO, int G>    // G lanes a channel (a power of two): N <= 8 G
__global__ void __launch_bounds__(128) selective_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    pdl_wait();
    constexpr int CPW = 32 / G;
    const int CPB = (blockDim.x >> 5) * CPW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % G;
    const int cl = warp * CPW + lane / G;              // channel within the block
    const int c0 = blockIdx.x * CPB;
    const bool live = c0 + cl < a.C;
    const int c = live ? c0 + cl : a.C - 1;
    const int b = blockIdx.y;
    const int first = a.row_offsets[b], end = a.row_offsets[b + 1];
    const int N = a.N, n0 = sub * SCAN_NPT, NP = G * SCAN_NPT;
    // one buffer: [CH][4][CPB] (dt | dt x | D x | gate) then [CH][2][NP] (B | C)
    const int CH = a.ch;
    const int buf_floats = CH * (4 * CPB + 2 * NP);
    float* S_g = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)c * N;
    float S[SCAN_NPT], A[SCAN_NPT];
    const bool vec = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(S_g) & 15) == 0);
    if (vec) {
#pragma unroll
        for (int i = 0; i < SCAN_NPT; i += 4) {
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (n0 + i < N) v = *reinterpret_cast<const float4*>(S_g + n0 + i);
            S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i) S[i] = n0 + i < N ? S_g[n0 + i] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < SCAN_NPT; ++i)
        A[i] = n0 + i < N ? -expf(a.a_log[(size_t)c * N + n0 + i]) * 1.4426950408889634f : 0.0f;
    // states beyond N stay zero in both buffers' B and C
    if (NP != N) for (int i = threadIdx.x; i < SCAN_STAGES * buf_floats; i += blockDim.x) {
        const int within = i % buf_floats, row_part = within % (4 * CPB + 2 * NP);
        if (row_part >= 4 * CPB && (row_part - 4 * CPB) % NP >= N) sm[i] = 0.0f;
    }
    const int live_ch = min(CPB, a.C - c0);
    auto fetch = [&](int t0, int buf) {
        const int rows = max(0, min(CH, end - t0));           // none: an empty group keeps the count of groups even
        float* base = sm + buf * buf_floats;
        const int stride = 4 * CPB + 2 * NP;
        if (a.vec_ch) {
            const int q = live_ch >> 2;
            for (int i = threadIdx.x; i < rows * q; i += blockDim.x) {
                const int tt = i / q, ch = (i % q) * 4;
                float* row = base + tt * stride;
                const size_t t = (size_t)(t0 + tt);
                cp_async16(row + ch, a.dtraw + t * a.C + c0 + ch);
                cp_async16(row + CPB + ch, a.x + t * a.C + c0 + ch);
                cp_async16(row + 3 * CPB + ch, a.z + t * a.ld_z + c0 + ch);
            }
        } else {
            for (int i = threadIdx.x; i < rows * live_ch; i += blockDim.x) {
                const int tt = i / live_ch, ch = i % live_ch;
                float* row = base + tt * stride;
                const size_t t = (size_t)(t0 + tt);
                cp_async4(row + ch, a.dtraw + t * a.C + c0 + ch);
                cp_async4(row + CPB + ch, a.x + t * a.C + c0 + ch);
                cp_async4(row + 3 * CPB + ch, a.z + t * a.ld_z + c0 + ch);
            }
        }
        if (a.vec_bc) {
            const int q = N >> 2;
            for (int i = threadIdx.x; i < rows * q; i += blockDim.x) {
                const int tt = i / q, n = (i % q) * 4;
                float* row = base + tt * stride + 4 * CPB;
                const float* src = a.bc + (size_t)(t0 + tt) * a.ld_bc;
                cp_async16(row + n, src + a.col_b + n);
                cp_async16(row + NP + n, src + a.col_c + n);
            }
        } else {
            for (int i = threadIdx.x; i < rows * N; i += blockDim.x) {
                const int tt = i / N, n = i % N;
                float* row = base + tt * stride + 4 * CPB;
                const float* src = a.bc + (size_t)(t0 + tt) * a.ld_bc;
                cp_async4(row + n, src + a.col_b + n);
                cp_async4(row + NP + n, src + a.col_c + n);
            }
        }
        cp_async_commit();
    };
    fetch(first, 0);
    fetch(first + CH, 1);
    int buf = 0;
    for (int t0 = first; t0 < end; t0 += CH, buf = (buf + 1) % SCAN_STAGES) {
        const int rows = min(CH, end - t0);
        cp_async_wait<1>();       // all but the newest group: this chunk is here
        __syncthreads();          // ... for everyone, and everyone has left the chunk before
        fetch(t0 + 2 * CH, (buf + 2) % SCAN_STAGES);         // two chunks ahead, into the buffer of the chunk before
        const float* base = sm + buf * buf_floats;
        const float dsk = a.dskip[c];
#pragma unroll 1
        for (int tt = 0; tt < rows; ++tt) {
            const float* row = base + tt * (4 * CPB + 2 * NP);
            const float dt = row[cl], xv = row[CPB + cl], dtx = dt * xv;
            const float4* B4 = reinterpret_cast<const float4*>(row + 4 * CPB + n0);
            const float4* C4 = reinterpret_cast<const float4*>(row + 4 * CPB + NP + n0);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_NPT / 4; ++i) {
                const float4 Bv = B4[i], Cv = C4[i];
                S[4 * i] = fmaf(ex2_approx(dt * A[4 * i]), S[4 * i], dtx * Bv.x);             acc = fmaf(S[4 * i], Cv.x, acc);
                S[4 * i + 1] = fmaf(ex2_approx(dt * A[4 * i + 1]), S[4 * i + 1], dtx * Bv.y); acc = fmaf(S[4 * i + 1], Cv.y, acc);
                S[4 * i + 2] = fmaf(ex2_approx(dt * A[4 * i + 2]), S[4 * i + 2], dtx * Bv.z); acc = fmaf(S[4 * i + 2], Cv.z, acc);
                S[4 * i + 3] = fmaf(ex2_approx(dt * A[4 * i + 3]), S[4 * i + 3], dtx * Bv.w); acc = fmaf(S[4 * i + 3], Cv.w, acc);
            }
#pragma unroll
            for (int o = G >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && sub == 0)
                ((TO*)a.out)[(size_t)(t0 + tt) * a.C + c] = from_float<TO>(fmaf(dsk, xv, acc) * row[3 * CPB + cl]);
        }
    }
    if (live) {
        if (vec) {
#pragma unroll
            for (int i = 0; i < SCAN_NPT; i += 4)
                if (n0 + i < N) *reinterpret_cast<float4*>(S_g + n0 + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < SCAN_NPT; ++i)
                if (n0 + i < N) S_g[n0 + i] = S[i];
        }
    }
}

template <typename TO>
static int launch_scan(ScanArgs a, int B, int T, cudaStream_t stream) {
    int G = 1;
    while (G * SCAN_NPT < a.N) G <<= 1;
    if (G > 32) return SHARPI_BAD_ARGUMENT;
    int warps = 4;
    if ((long long)((a.C + 4 * (32 / G) - 1) / (4 * (32 / G))) * B < 296) warps = 1;     // too few blocks for 148 SMs
    const int cpb = warps * (32 / G);
    const dim3 grid((a.C + cpb - 1) / cpb, B);
    a.ch = T - B + 1 < SCAN_CH ? (T - B + 1 < 1 ? 1 : T - B + 1) : SCAN_CH;    // no request brings more rows than T - B + 1
    const size_t smem = (size_t)SCAN_STAGES * a.ch * (4 * cpb + 2 * G * SCAN_NPT) * sizeof(float);
    const uintptr_t chp = reinterpret_cast<uintptr_t>(a.dtraw) | reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.z);
    a.vec_ch = (a.C % 4 == 0 && cpb % 4 == 0 && a.ld_z % 4 == 0 && (chp & 15) == 0) ? 1 : 0;
    a.vec_bc = (a.N % 4 == 0 && a.col_b % 4 == 0 && a.col_c % 4 == 0 && a.ld_bc % 4 == 0 &&
                (reinterpret_cast<uintptr_t>(a.bc) & 15) == 0) ? 1 : 0;
#define SCAN_CASE(GG)                                                                                          \
    case GG: {                                                                                                 \
        auto kern = selective_scan_kernel<TO, GG>;                                                             \
        if (smem > 48 * 1024 &&                                                                                \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return SHARPI_LAUNCH_FAILED;                                                                       \
        SHARPI_LAUNCH_PDL(kern, grid, warps * 32, smem, stream, a);                                            \
        break;                                                                                                 \
    }
    switch (G) {
        SCAN_CASE(1) SCAN_CASE(2) SCAN_CASE(4) SCAN_CASE(8) SCAN_CASE(16) SCAN_CASE(32)
        default: return SHARPI_BAD_ARGUMENT;
    }
#undef SCAN_CASE
    return SHARPI_OK;
}

SHARPI_API int sharpi_selective_scan(const float* x, const float* dtraw, const float* bc,
                                     int ld_bc, int col_b, int col_c, const float* a_log, const float* dskip,
                                     const float* z, int ld_z, const int* row_offsets, const int* state_slots,
                                     float* state, long long state_stride, void* out, int out_dtype, int T, int B,
                                     int C, int N, cudaStream_t stream) {
    if (B <= 0) return SHARPI_OK;
    if (C <= 0 || N <= 0 || N > 256) return SHARPI_BAD_ARGUMENT;
    ScanArgs a;
    a.x = x; a.dtraw = dtraw; a.bc = bc; a.ld_bc = ld_bc; a.col_b = col_b; a.col_c = col_c;
    a.a_log = a_log; a.dskip = dskip; a.z = z; a.ld_z = ld_z; a.row_offsets = row_offsets; a.state_slots = state_slots;
    a.state = state; a.state_stride = state_stride; a.out = out; a.C = C; a.N = N;
    if (out_dtype == SHARPI_F32) return launch_scan<float>(a, B, T, stream);
    if (out_dtype == SHARPI_BF16) return launch_scan<bf16>(a, B, T, stream);
    return SHARPI_BAD_ARGUMENT;
}
