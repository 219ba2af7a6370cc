// A selective state-space mixer's two kernels: the short causal convolution with its activation, and the scan.
//
// Per sequence and channel c the mixer keeps, in a float32 state row [slots][stride]:
//   S[c][n], n < N          at c * N + n                       the recurrence's state
//   the last K - 1 inputs   at conv_off + i * channels + c     of the convolution, oldest first (i = 0 .. K - 2)
// Both are zero when a sequence starts, so a tap that reaches before the first token meets a zero.
//
//   conv:  u[t][c] = silu(bias[c] + sum_k w[c][k] x[t - (K - 1 - k)][c])      (the last column of w meets the current token)
//   scan:  dt = softplus(dt_raw[t][c] + dt_bias[c])
//          S[c][n] = exp(dt A[c][n]) S[c][n] + dt u[t][c] B[t][n]
//          y[t][c] = (sum_n S[c][n] C[t][n] + D[c] u[t][c]) * silu(z[t][c])
//
// Step sizes, decays, states and every sum are float32 whatever the activation type.  One device function makes a token's
// step, for prompts and for one-token steps alike, and the sums over n run in an order that depends on N only (a thread's
// own states in ascending order, then the threads of a channel as a shuffle tree; how many threads share a channel depends on N alone), so a token's result is the same bits
// however its sequence was cut into passes and whatever else the pass holds.
#include "common.cuh"

#define SSM_THREADS 128    // per block of the scan: channels x the threads that share a channel's states
#define SSM_TC 32          // tokens staged at a time
#define SSM_MAX_TAPS 16

// exp(a * b) for a * b <= 0, closer than the library's exponential (whose error of up to two units in the last place, met
// again at every token, is what a slowly decaying state adds up): the product's own rounding error is carried along
// (x_lo), x = n ln2 + r with ln2 in two parts, and exp(r) is a polynomial of degree 7 over |r| <= ln2 / 2, all in fused
// multiply-adds.  Below 2^-126 the result is zero.
__device__ __forceinline__ float ssm_exp_prod(float a, float b) {
    const float x = a * b;
    const float x_lo = fmaf(a, b, -x);
    const float n = rintf(x * 1.4426950408889634f);
    if (n < -126.f) return 0.f;
    float r = fmaf(n, -0.693145751953125f, x);           // ln2's leading bits: n times it is exact
    r = fmaf(n, -1.428606765330187e-06f, r) + x_lo;
    float p = 1.98412698e-4f;                             // 1/7!
    p = fmaf(p, r, 1.38888889e-3f);
    p = fmaf(p, r, 8.33333333e-3f);
    p = fmaf(p, r, 4.16666667e-2f);
    p = fmaf(p, r, 1.66666667e-1f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    return p * __int_as_float(((int)n + 127) << 23);
}

__device__ __forceinline__ float ssm_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float ssm_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ----------------------------------------------------------------------------------------
// Convolution.  One thread per (row, channel).  The inputs before a row are the rows above it in the pass while they
// belong to the same sequence (same slot, positions that count down by one), and the sequence's kept inputs beyond.
// The state is only read here: the scan, which runs later in the stream, leaves the new last inputs.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int64_t ld, const float* __restrict__ w, const float* __restrict__ bias,
                                        const float* __restrict__ state, int64_t state_stride, int64_t conv_off, T* __restrict__ out,
                                        const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos, int n_rows,
                                        int channels, int taps) {
    pdl_launch_dependents();
    const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int row = (int)(item / channels), c = (int)(item % channels);
    float wk[SSM_MAX_TAPS];
    float b = 0.f;
    if (row < n_rows) {
#pragma unroll
        for (int k = 0; k < SSM_MAX_TAPS; ++k) wk[k] = k < taps ? w[(int64_t)c * taps + k] : 0.f;
        b = bias != nullptr ? bias[c] : 0.f;
    }
    pdl_wait();
    if (row >= n_rows) return;
    const int slot = row_slot[row], pos = row_pos[row];
    // how many rows right above this one continue its sequence (at most K - 1 are looked at)
    int above = 0;
    while (above < taps - 1 && row - above - 1 >= 0 && row_slot[row - above - 1] == slot && row_pos[row - above - 1] == pos - above - 1) ++above;
    float acc = b;
#pragma unroll
    for (int k = 0; k < SSM_MAX_TAPS; ++k) {
        if (k >= taps) break;
        const int back = taps - 1 - k;          // this tap meets the input `back` tokens ago
        float v = 0.f;
        if (back <= above) v = to_f32(x[(int64_t)(row - back) * ld + c]);
        else if (slot >= 0) v = state[(int64_t)slot * state_stride + conv_off + (int64_t)(taps - 1 + above - back) * channels + c];
        acc = fmaf(wk[k], v, acc);
    }
    out[(int64_t)row * channels + c] = from_f32<T>(ssm_silu(acc));
}

// The same for 8 consecutive channels per thread (channels and row pitch multiples of 8, 16-byte aligned rows): 16-byte
// loads and stores; a channel's sum runs over the taps in the same order, so it has the same bits.
__device__ __forceinline__ void ssm_load8(const float* p, float* v) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ssm_load8(const bf16* p, float* v) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void ssm_store8(float* p, const float* v) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void ssm_store8(bf16* p, const float* v) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

#define SSM_CONV_ROWS 16        // rows a block of the vectorised convolution walks with its taps staged once (one row in short passes)
#define SSM_CONV_VEC_TAPS 8     // most taps that kernel stages

template <typename T>
__global__ void __launch_bounds__(128) causal_conv_silu_vec_kernel(
        const T* __restrict__ x, int64_t ld, const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
        int64_t state_stride, int64_t conv_off, T* __restrict__ out, const int32_t* __restrict__ row_slot,
        const int32_t* __restrict__ row_pos, int n_rows, int channels, int taps, int rows_per_block) {
    // the taps of this block's 128 x 8 channels, laid out [tap][channel of the thread's eight][thread]: a warp's reads of
    // one (tap, channel) are 32 consecutive words
    __shared__ float w_s[SSM_CONV_VEC_TAPS * 8 * 128];
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int c0 = blockIdx.x * 1024;
    for (int e = tid; e < 1024 * taps; e += 128) {              // e = channel of the block x taps + tap: the order they are stored in
        const int ch = e / taps, k = e - ch * taps;
        w_s[(k * 8 + (ch & 7)) * 128 + (ch >> 3)] = c0 + ch < channels ? w[(int64_t)(c0 + ch) * taps + k] : 0.f;
    }
    const int c = c0 + tid * 8;
    float b8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) b8[i] = 0.f;
    if (c < channels && bias != nullptr) ssm_load8(bias + c, b8);
    __syncthreads();
    pdl_wait();
    if (c >= channels) return;
    const int r_end = min(n_rows, (int)(blockIdx.y + 1) * rows_per_block);
    for (int row = blockIdx.y * rows_per_block; row < r_end; ++row) {
        const int slot = row_slot[row], pos = row_pos[row];
        int above = 0;
        while (above < taps - 1 && row - above - 1 >= 0 && row_slot[row - above - 1] == slot && row_pos[row - above - 1] == pos - above - 1) ++above;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = b8[i];
        for (int k = 0; k < taps; ++k) {
            const int back = taps - 1 - k;
            float v[8];
            if (back <= above) ssm_load8(x + (int64_t)(row - back) * ld + c, v);
            else if (slot >= 0) ssm_load8(state + (int64_t)slot * state_stride + conv_off + (int64_t)(taps - 1 + above - back) * channels + c, v);
            else
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(w_s[(k * 8 + i) * 128 + tid], v[i], acc[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = ssm_silu(acc[i]);
        ssm_store8(out + (int64_t)row * channels + c, acc);
    }
}

X0NE_API int x0ne_causal_conv_silu(const void* x, int64_t ld, int dt, const float* w, const float* bias, const float* state,
                                   int64_t state_stride, int64_t conv_off, void* out, const int32_t* row_slot, const int32_t* row_pos,
                                   int n_rows, int channels, int taps, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && channels > 0 && taps >= 1 && taps <= SSM_MAX_TAPS && ld >= channels,
                 "causal_conv: rows %d channels %d taps %d (at most %d)", n_rows, channels, taps, SSM_MAX_TAPS);
    X0NE_REQUIRE(conv_off >= 0 && state_stride >= conv_off + (int64_t)(taps - 1) * channels, "causal_conv: the state row is too short");
    if (n_rows == 0) return 0;
    if (channels % 8 == 0 && ld % 8 == 0 && conv_off % 4 == 0 && state_stride % 4 == 0 && (dt == X0NE_F32 || dt == X0NE_BF16) &&
        taps <= SSM_CONV_VEC_TAPS && n_rows <= 65535 * SSM_CONV_ROWS &&
        ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)state | (uintptr_t)bias) & 15) == 0)) {
        const int rpb = n_rows >= 256 ? SSM_CONV_ROWS : 1;
        const dim3 vgrid((unsigned)((channels + 1023) / 1024), (unsigned)((n_rows + rpb - 1) / rpb));
        if (dt == X0NE_F32)
            x0ne_launch(causal_conv_silu_vec_kernel<float>, vgrid, dim3(128), 0, stream, (const float*)x, ld, w, bias, state, state_stride, conv_off,
                        (float*)out, row_slot, row_pos, n_rows, channels, taps, rpb);
        else
            x0ne_launch(causal_conv_silu_vec_kernel<bf16>, vgrid, dim3(128), 0, stream, (const bf16*)x, ld, w, bias, state, state_stride, conv_off,
                        (bf16*)out, row_slot, row_pos, n_rows, channels, taps, rpb);
        X0NE_LAUNCH_CHECK();
    }
    const int64_t items = (int64_t)n_rows * channels;
    const dim3 grid((unsigned)((items + 255) / 256));
    if (dt == X0NE_F32)
        x0ne_launch(causal_conv_silu_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ld, w, bias, state, state_stride, conv_off,
                    (float*)out, row_slot, row_pos, n_rows, channels, taps);
    else if (dt == X0NE_BF16)
        x0ne_launch(causal_conv_silu_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ld, w, bias, state, state_stride, conv_off,
                    (bf16*)out, row_slot, row_pos, n_rows, channels, taps);
    else
        X0NE_REQUIRE(false, "causal_conv: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Scan.  A block takes one sequence and 128 / SSM_SPLIT channels; SSM_SPLIT threads share a channel, each with NS states
// (n = part * NS + i) in registers.  The sequence's rows are staged SSM_TC at a time: all threads fetch the next tokens'
// values into registers while the block works through the staged ones, then turn them into what the step needs
// (softplus, silu) on their way to shared memory.  Only S is carried from token to token: the decays of U tokens are
// worked out side by side, and the state's own chain is one fused multiply-add per token and value.
// ----------------------------------------------------------------------------------------
struct SsmArgs {
    const void* u;            // [rows][channels], activation type: the convolution's output
    const void* xz;           // [rows][xz_ld], activation type: the convolution's input at column 0, z at column z_col
    int64_t xz_ld;
    int32_t z_col;
    const float* dt_raw;      // [rows][channels]
    const float* dt_bias;     // [channels] or null
    const float* A;           // [channels][N], negative
    const float* bc;          // [rows][bc_ld]: B at b_col, C at c_col
    int64_t bc_ld;
    int32_t b_col, c_col;
    const float* D;           // [channels] or null
    void* out;                // [rows][channels], activation type
    float* state;
    int64_t state_stride, conv_off;
    const int32_t* seq_first_row;
    const int32_t* seq_slot;
    int32_t channels, N, taps;
};

// What the scan works out per token, by the run's type.  float32 runs take the close exponential above and the library's
// softplus and sigmoid; bfloat16 runs, whose inputs carry eight bits, the hardware's exponential, logarithm and
// reciprocal (float32 all the same: errors near 2^-21).
template <typename T> struct SsmMath;
template <> struct SsmMath<float> {
    static __device__ __forceinline__ float decay(float dt, float a) { return ssm_exp_prod(dt, a); }
    static __device__ __forceinline__ float softplus(float v) { return ssm_softplus(v); }
    static __device__ __forceinline__ float silu(float v) { return ssm_silu(v); }
};
template <> struct SsmMath<bf16> {
    static __device__ __forceinline__ float decay(float dt, float a) { return __expf(dt * a); }
    static __device__ __forceinline__ float softplus(float v) { return v > 15.f ? v : __logf(1.0f + __expf(v)); }
    static __device__ __forceinline__ float silu(float v) { return v * __frcp_rn(1.0f + __expf(-v)); }
};

// The last K - 1 inputs of a sequence's convolution after a pass of n_tok rows from row0: rows of the pass, and, where the
// pass brought fewer, the kept ones moved up.  One thread per channel.
template <typename T>
__device__ __forceinline__ void ssm_keep_inputs(const SsmArgs& a, float* st, const T* xz, int row0, int n_tok, int c) {
    if (a.taps <= 1) return;
    float keep[SSM_MAX_TAPS];
    const int kept = a.taps - 1;
#pragma unroll
    for (int i = 0; i < SSM_MAX_TAPS; ++i) {
        if (i >= kept) break;
        const int t = n_tok - kept + i;         // the token of this pass that belongs at place i (negative: an older one)
        keep[i] = t >= 0 ? to_f32(xz[(int64_t)(row0 + t) * a.xz_ld + c]) : st[a.conv_off + (int64_t)(i + n_tok) * a.channels + c];
    }
#pragma unroll
    for (int i = 0; i < SSM_MAX_TAPS; ++i) {
        if (i >= kept) break;
        st[a.conv_off + (int64_t)i * a.channels + c] = keep[i];
    }
}

// A pass in which every sequence brings one row (or few): a thread reads its token's values itself, nothing is staged and
// no thread waits for another.  The operations of a token and their order are the staged kernel's, so the bits are.
template <typename T, int NS, int SSM_SPLIT>
__global__ void __launch_bounds__(SSM_THREADS) selective_scan_step_kernel(SsmArgs a) {
    constexpr int SSM_CH = SSM_THREADS / SSM_SPLIT;
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int cl = tid / SSM_SPLIT, part = tid % SSM_SPLIT;
    const int c = blockIdx.x * SSM_CH + cl;
    const int seq = blockIdx.y;
    const bool live = c < a.channels;
    float An[NS], S[NS];
    float Dc = 0.f, dtb = 0.f;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        An[i] = live && n < a.N ? a.A[(int64_t)c * a.N + n] : 0.f;
    }
    if (live) {
        Dc = a.D != nullptr ? a.D[c] : 0.f;
        dtb = a.dt_bias != nullptr ? a.dt_bias[c] : 0.f;
    }
    pdl_wait();
    const int slot = a.seq_slot[seq];
    const int row0 = a.seq_first_row[seq], n_tok = a.seq_first_row[seq + 1] - row0;
    if (slot < 0 || n_tok <= 0) return;
    float* st = a.state + (int64_t)slot * a.state_stride;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        S[i] = live && n < a.N ? st[(int64_t)c * a.N + n] : 0.f;
    }
    const T* u = (const T*)a.u;
    const T* xz = (const T*)a.xz;
    T* out = (T*)a.out;
    for (int t = 0; t < n_tok; ++t) {
        const int64_t r = row0 + t;
        const float dt = live ? SsmMath<T>::softplus(a.dt_raw[r * a.channels + c] + dtb) : 0.f;
        const float uv = live ? to_f32(u[r * a.channels + c]) : 0.f;
        const float dtu = dt * uv;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            const int n = part * NS + i;
            const float bn = n < a.N ? a.bc[r * a.bc_ld + a.b_col + n] : 0.f, cn = n < a.N ? a.bc[r * a.bc_ld + a.c_col + n] : 0.f;
            S[i] = fmaf(SsmMath<T>::decay(dt, An[i]), S[i], dtu * bn);
            acc = fmaf(S[i], cn, acc);
        }
#pragma unroll
        for (int w = 1; w < SSM_SPLIT; w <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
        if (part == 0 && live)
            out[r * a.channels + c] = from_f32<T>(fmaf(Dc, uv, acc) * SsmMath<T>::silu(to_f32(xz[r * a.xz_ld + a.z_col + c])));
    }
    if (!live) return;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        if (n < a.N) st[(int64_t)c * a.N + n] = S[i];
    }
    if (part == 0) ssm_keep_inputs<T>(a, st, xz, row0, n_tok, c);
}

template <typename T, int NS, int SSM_SPLIT, int U>
__global__ void __launch_bounds__(SSM_THREADS) selective_scan_kernel(SsmArgs a) {
    constexpr int THREADS = SSM_THREADS;
    constexpr int SSM_CH = THREADS / SSM_SPLIT;                 // channels per block
    constexpr int NP = NS * SSM_SPLIT;                          // states per channel as the block holds them
    constexpr int PER_CH = (SSM_TC * SSM_CH + THREADS - 1) / THREADS;   // staged (token, channel) values per thread
    constexpr int PER_N = (SSM_TC * NP + THREADS - 1) / THREADS;
    __shared__ float s_dt[SSM_TC][SSM_CH], s_u[SSM_TC][SSM_CH], s_z[SSM_TC][SSM_CH];
    __shared__ __align__(16) float s_b[SSM_TC][NP], s_c[SSM_TC][NP];
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int cl = tid / SSM_SPLIT, part = tid % SSM_SPLIT;
    const int c = blockIdx.x * SSM_CH + cl;
    const int seq = blockIdx.y;
    const bool live = c < a.channels;
    float An[NS], S[NS];
    float Dc = 0.f;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        An[i] = live && n < a.N ? a.A[(int64_t)c * a.N + n] : 0.f;
    }
    if (live) Dc = a.D != nullptr ? a.D[c] : 0.f;
    // the staging thread's own (token, channel) and (token, n) places
    const int c_st = tid % SSM_CH, ch_st = blockIdx.x * SSM_CH + c_st;
    const float dtb_st = ch_st < a.channels && a.dt_bias != nullptr ? a.dt_bias[ch_st] : 0.f;
    pdl_wait();
    const int slot = a.seq_slot[seq];
    const int row0 = a.seq_first_row[seq], n_tok = a.seq_first_row[seq + 1] - row0;
    if (slot < 0 || n_tok <= 0) return;
    float* st = a.state + (int64_t)slot * a.state_stride;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        S[i] = live && n < a.N ? st[(int64_t)c * a.N + n] : 0.f;
    }
    const T* u = (const T*)a.u;
    const T* xz = (const T*)a.xz;
    T* out = (T*)a.out;

    // (fetched values stay as they were read until they are staged: an instruction that used one right away would hold the
    // warp until the read came back)
    float f_dt[PER_CH], f_b[PER_N], f_c[PER_N];
    T f_u[PER_CH], f_z[PER_CH];
    // rows of a stage that are fetched and staged: the sequence's own, and the few past its end that the last group of U
    // tokens reaches (they are staged as steps of zero)
    auto staged_end = [&](int t0) { return t0 + (min(n_tok - t0, SSM_TC) + U - 1) / U * U; };
    auto fetch = [&](int t0) {
        const int t_end = staged_end(t0);
#pragma unroll
        for (int j = 0; j < PER_CH; ++j) {
            if (t0 + j * (THREADS / SSM_CH) >= t_end) break;        // (the same for every thread: a short pass stages what it has)
            const int t = t0 + (tid / SSM_CH) + j * (THREADS / SSM_CH);
            const bool ok = t < t0 + SSM_TC && t < n_tok && ch_st < a.channels;
            const int64_t r = row0 + (ok ? t : 0);
            f_dt[j] = a.dt_raw[ok ? r * a.channels + ch_st : 0];
            f_u[j] = u[ok ? r * a.channels + ch_st : 0];
            f_z[j] = xz[ok ? r * a.xz_ld + a.z_col + ch_st : 0];
        }
#pragma unroll
        for (int j = 0; j < PER_N; ++j) {
            if (t0 + j * THREADS / NP >= t_end) break;
            const int e = tid + j * THREADS;
            const int t = t0 + e / NP, n = e % NP;
            const bool ok = e < SSM_TC * NP && t < n_tok && n < a.N;
            const int64_t r = row0 + (ok ? t : 0);
            f_b[j] = ok ? a.bc[r * a.bc_ld + a.b_col + n] : 0.f;      // (a state past N must read as zero)
            f_c[j] = ok ? a.bc[r * a.bc_ld + a.c_col + n] : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < n_tok; t0 += SSM_TC) {
        const int t_end = staged_end(t0);
#pragma unroll
        for (int j = 0; j < PER_CH; ++j) {
            if (t0 + j * (THREADS / SSM_CH) >= t_end) break;        // rows past those are not read: the walk below stops there
            const int tl = (tid / SSM_CH) + j * (THREADS / SSM_CH);
            if (tl < SSM_TC) {
                // a place past the sequence's last row gets a step of zero: it leaves the state as it is, bit for bit
                s_dt[tl][c_st] = t0 + tl < n_tok ? SsmMath<T>::softplus(f_dt[j] + dtb_st) : 0.f;
                s_u[tl][c_st] = t0 + tl < n_tok ? to_f32(f_u[j]) : 0.f;
                s_z[tl][c_st] = SsmMath<T>::silu(to_f32(f_z[j]));
            }
        }
#pragma unroll
        for (int j = 0; j < PER_N; ++j) {
            if (t0 + j * THREADS / NP >= t_end) break;
            const int e = tid + j * THREADS;
            if (e < SSM_TC * NP) {
                s_b[e / NP][e % NP] = f_b[j];
                s_c[e / NP][e % NP] = f_c[j];
            }
        }
        __syncthreads();
        if (t0 + SSM_TC < n_tok) fetch(t0 + SSM_TC);
        // U tokens at a time: their decays and inputs do not depend on the state, so they are worked out side by side;
        // the state then takes one fused multiply-add per token and value, in the tokens' order
#pragma unroll 1
        for (int tl0 = 0; tl0 < SSM_TC && t0 + tl0 < n_tok; tl0 += U) {
            float dec[U][NS], in[U][NS], uv[U], acc[U];
#pragma unroll
            for (int k = 0; k < U; ++k) {
                const float dt = s_dt[tl0 + k][cl];
                uv[k] = s_u[tl0 + k][cl];
                const float dtu = dt * uv[k];
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    dec[k][i] = SsmMath<T>::decay(dt, An[i]);
                    in[k][i] = dtu * s_b[tl0 + k][part * NS + i];
                }
            }
#pragma unroll
            for (int k = 0; k < U; ++k) {
                acc[k] = 0.f;
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    S[i] = fmaf(dec[k][i], S[i], in[k][i]);
                    acc[k] = fmaf(S[i], s_c[tl0 + k][part * NS + i], acc[k]);
                }
            }
#pragma unroll
            for (int w = 1; w < SSM_SPLIT; w <<= 1) {
#pragma unroll
                for (int k = 0; k < U; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], w);
            }
            if (part == 0 && live) {
#pragma unroll
                for (int k = 0; k < U; ++k)
                    if (t0 + tl0 + k < n_tok)
                        out[(int64_t)(row0 + t0 + tl0 + k) * a.channels + c] = from_f32<T>(fmaf(Dc, uv[k], acc[k]) * s_z[tl0 + k][cl]);
            }
        }
        __syncthreads();
    }
    if (!live) return;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = part * NS + i;
        if (n < a.N) st[(int64_t)c * a.N + n] = S[i];
    }
    if (part == 0) ssm_keep_inputs<T>(a, st, xz, row0, n_tok, c);
}

// How many threads share a channel: 4, 8 or 16 (more threads per channel are more warps to hide the latency of a token's
// dependent steps with, at more instructions in all; a single prompt's scan is bound by that latency, many sequences'
// by the instructions).
// A float32 run's choice depends on N alone, so that a token has the same bits in every pass; a bfloat16 run takes the
// fewest threads per channel that still give every scheduler of the GPU a few warps.
template <typename T>
static int selective_scan_launch(const SsmArgs& a, int n_seqs, int sm_count, int one_token, cudaStream_t stream) {
    int split = a.N > 32 ? 16 : 4;
    if (sizeof(T) == 2) {
        const int64_t want_warps = (int64_t)sm_count * 4 * 3;
        while (split < 16 && split < a.N && (int64_t)n_seqs * a.channels * split / 32 < want_warps) split *= 2;
    }
    const int ns = (a.N + split - 1) / split;
    const dim3 grid((unsigned)((a.channels + SSM_THREADS / split - 1) / (SSM_THREADS / split)), (unsigned)n_seqs), block(SSM_THREADS);
    // (a pass in which every sequence brings one row takes the kernel that stages nothing)
#define SSM_GO(NS, SPLIT, U)                                                                                   \
    do {                                                                                                       \
        if (one_token) x0ne_launch(selective_scan_step_kernel<T, NS, SPLIT>, grid, block, 0, stream, a);       \
        else x0ne_launch(selective_scan_kernel<T, NS, SPLIT, U>, grid, block, 0, stream, a);                   \
    } while (0)
    if (split == 4) {
        if (ns <= 1) SSM_GO(1, 4, 4);
        else if (ns <= 2) SSM_GO(2, 4, 4);
        else if (ns <= 4) SSM_GO(4, 4, 4);
        else if (ns <= 6) SSM_GO(6, 4, 2);
        else SSM_GO(8, 4, 2);
    } else if (split == 8) {
        if (ns <= 1) SSM_GO(1, 8, 4);
        else if (ns <= 2) SSM_GO(2, 8, 4);
        else SSM_GO(4, 8, 2);
    } else {
        if (ns <= 1) SSM_GO(1, 16, 4);
        else if (ns <= 2) SSM_GO(2, 16, 4);
        else if (ns <= 3) SSM_GO(3, 16, 2);
        else if (ns <= 4) SSM_GO(4, 16, 2);
        else if (ns <= 6) SSM_GO(6, 16, 1);
        else SSM_GO(8, 16, 1);
    }
#undef SSM_GO
    X0NE_LAUNCH_CHECK();
}

X0NE_API int x0ne_selective_scan(SsmArgs a, int dt, int n_seqs, int one_token, cudaStream_t stream) {
    X0NE_REQUIRE(n_seqs >= 0 && n_seqs <= 65535 && a.channels > 0 && a.N > 0 && a.N <= 128 && a.taps >= 1 && a.taps <= SSM_MAX_TAPS,
                 "selective_scan: %d sequences, %d channels of %d states (at most %d), %d taps", n_seqs, a.channels, a.N, 128, a.taps);
    X0NE_REQUIRE(a.conv_off >= (int64_t)a.channels * a.N && a.state_stride >= a.conv_off + (int64_t)(a.taps - 1) * a.channels,
                 "selective_scan: the state row is too short");
    X0NE_REQUIRE(a.xz_ld >= a.channels && a.z_col >= 0 && a.z_col + a.channels <= a.xz_ld && a.b_col >= 0 && a.c_col >= 0 &&
                     a.b_col + a.N <= a.bc_ld && a.c_col + a.N <= a.bc_ld, "selective_scan: columns lie outside their rows");
    if (n_seqs == 0) return 0;
    static int sm_count[64] = {};
    const int dev = OncePerDevice::device();
    int sms = dev >= 0 ? sm_count[dev] : 0;
    if (sms <= 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev >= 0 ? dev : 0) != cudaSuccess || sms <= 0) sms = 148;
        if (dev >= 0) sm_count[dev] = sms;
    }
    if (dt == X0NE_F32) return selective_scan_launch<float>(a, n_seqs, sms, one_token, stream);
    if (dt == X0NE_BF16) return selective_scan_launch<bf16>(a, n_seqs, sms, one_token, stream);
    X0NE_REQUIRE(false, "selective_scan: unknown dtype tag %d", dt);
}
