// The selective state-space scan (Mamba) from per-request state, and the short causal convolution before it.
//
//   sharpi_causal_conv   x_t[c] = silu(b[c] + sum_j w[c][j] in_{t - (taps - 1 - j)}[c]): the last column of w is
//                        the current token's.  Inputs before a portion's first row come from the request's state
//                        (its last taps - 1 inputs; zeros at a sequence's start), which a second launch then
//                        moves on to the portion's last inputs.
//   sharpi_slice_cols    a block of columns of a float32 matrix as a contiguous matrix in the activation dtype
//                        (the step-size inputs of the scan, cut out of the fused projection).
//   sharpi_selective_scan  per channel c and state n, for the rows of a request in order:
//                            dt = softplus(dtraw[c] + dt_bias[c])
//                            S[c][n] <- exp(dt A[c][n]) S[c][n] + dt x[c] B[n],  A = -exp(A_log)
//                            y[c] = sum_n S[c][n] C[n] + D[c] x[c],  out = y silu(z[c])
//                        all in float32.  A group of lanes owns one channel, each lane eight states in registers;
//                        the sum over the states is a fixed tree of exchanges, and the walk over a request's rows
//                        is sequential, so a row's result does not depend on how the prompt was cut or batched.
#include "common.cuh"

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* in, int ld, const float* __restrict__ w, const float* __restrict__ bias,
                   const float* state, long long state_stride, const int* row_request, const int* row_offsets,
                   const int* state_slots, float* x32, TO* xact, int C, int taps) {
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
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
                                  int taps, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (C <= 0 || taps <= 0 || B <= 0) return SHARPI_BAD_ARGUMENT;
    const dim3 grid(T, (C + 255) / 256);
    if (act_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(causal_conv_kernel<float>, grid, 256, 0, stream, in, ld, w, bias, (const float*)state,
                          state_stride, row_request, row_offsets, state_slots, x32, (float*)nullptr, C, taps);
    else if (act_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(causal_conv_kernel<bf16>, grid, 256, 0, stream, in, ld, w, bias, (const float*)state,
                          state_stride, row_request, row_offsets, state_slots, x32, (bf16*)xact, C, taps);
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
    const float* dtraw;      // [T, C]
    const float* dt_bias;    // [C]
    const float* bc;         // [T, ld_bc]: B at col_b, C at col_c, N columns each
    int ld_bc, col_b, col_c;
    const float* a_log;      // [C, N]
    const float* dskip;      // [C]
    const float* z;          // [T, ld_z]: the gate's input
    int ld_z;
    const int* row_offsets;
    const int* state_slots;
    float* state;            // [slots, C * N]
    long long state_stride;
    void* out;               // [T, C]
    int C, N;
};

constexpr int SCAN_NPT = 8;      // states a lane keeps

template <typename TO, int G>    // G lanes a channel (a power of two): N <= 8 G
__global__ void __launch_bounds__(128) selective_scan_kernel(ScanArgs a) {
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int CPW = 32 / G;                        // channels a warp
    const int sub = lane % G;
    const int c_raw = (blockIdx.x * (blockDim.x >> 5) + warp) * CPW + lane / G;
    const bool live = c_raw < a.C;
    const int c = live ? c_raw : a.C - 1;
    const int b = blockIdx.y;
    const int first = a.row_offsets[b], end = a.row_offsets[b + 1];
    const int N = a.N, n0 = sub * SCAN_NPT;
    float* S_g = a.state + (size_t)a.state_slots[b] * a.state_stride + (size_t)c * N;
    float S[SCAN_NPT], A[SCAN_NPT];
#pragma unroll
    for (int i = 0; i < SCAN_NPT; ++i) {
        const bool in = n0 + i < N;
        S[i] = in ? S_g[n0 + i] : 0.0f;
        A[i] = in ? -expf(a.a_log[(size_t)c * N + n0 + i]) : 0.0f;
    }
    const float bias = a.dt_bias[c], dsk = a.dskip[c];
    for (int t = first; t < end; ++t) {
        const float raw = a.dtraw[(size_t)t * a.C + c] + bias;
        const float dt = raw > 20.0f ? raw : log1pf(expf(raw));
        const float xv = a.x[(size_t)t * a.C + c];
        const float dtx = dt * xv;
        const float* bc = a.bc + (size_t)t * a.ld_bc;
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i) {
            const bool in = n0 + i < N;
            const float Bn = in ? bc[a.col_b + n0 + i] : 0.0f;
            const float Cn = in ? bc[a.col_c + n0 + i] : 0.0f;
            S[i] = expf(dt * A[i]) * S[i] + dtx * Bn;
            acc += S[i] * Cn;
        }
#pragma unroll
        for (int o = G >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (live && sub == 0) {
            const float zv = a.z[(size_t)t * a.ld_z + c];
            ((TO*)a.out)[(size_t)t * a.C + c] = from_float<TO>((acc + dsk * xv) * silu_f(zv));
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i)
            if (n0 + i < N) S_g[n0 + i] = S[i];
    }
}

template <typename TO>
static int launch_scan(const ScanArgs& a, int B, cudaStream_t stream) {
    int G = 1;
    while (G * SCAN_NPT < a.N) G <<= 1;
    if (G > 32) return SHARPI_BAD_ARGUMENT;
    const int cpb = 4 * (32 / G);                      // channels a block of four warps
    const dim3 grid((a.C + cpb - 1) / cpb, B);
#define SCAN_CASE(GG)                                                                        \
    case GG: SHARPI_LAUNCH_PDL((selective_scan_kernel<TO, GG>), grid, 128, 0, stream, a); break;
    switch (G) {
        SCAN_CASE(1) SCAN_CASE(2) SCAN_CASE(4) SCAN_CASE(8) SCAN_CASE(16) SCAN_CASE(32)
        default: return SHARPI_BAD_ARGUMENT;
    }
#undef SCAN_CASE
    return SHARPI_OK;
}

SHARPI_API int sharpi_selective_scan(const float* x, const float* dtraw, const float* dt_bias, const float* bc,
                                     int ld_bc, int col_b, int col_c, const float* a_log, const float* dskip,
                                     const float* z, int ld_z, const int* row_offsets, const int* state_slots,
                                     float* state, long long state_stride, void* out, int out_dtype, int B, int C,
                                     int N, cudaStream_t stream) {
    if (B <= 0) return SHARPI_OK;
    if (C <= 0 || N <= 0 || N > 256) return SHARPI_BAD_ARGUMENT;
    ScanArgs a;
    a.x = x; a.dtraw = dtraw; a.dt_bias = dt_bias; a.bc = bc; a.ld_bc = ld_bc; a.col_b = col_b; a.col_c = col_c;
    a.a_log = a_log; a.dskip = dskip; a.z = z; a.ld_z = ld_z; a.row_offsets = row_offsets; a.state_slots = state_slots;
    a.state = state; a.state_stride = state_stride; a.out = out; a.C = C; a.N = N;
    if (out_dtype == SHARPI_F32) return launch_scan<float>(a, B, stream);
    if (out_dtype == SHARPI_BF16) return launch_scan<bf16>(a, B, stream);
    return SHARPI_BAD_ARGUMENT;
}
