// A linear recurrence with a matrix state per head (time mixing in the manner of RWKV), in three kernels:
//
//   token shift   mix_s[row] = h[row] + (h_before[row] - h[row]) * mu_s  for s = 0 .. n_mix-1, where h_before
//                 is the row of the token before it in its sequence: the row above in the pass, or, for the
//                 first row a sequence brings, the row the sequence's state keeps (zeros at a sequence's start)
//   scan          per sequence and head, token by token over the rows the sequence brings, from the state S
//                 [N key channels][N value channels] the sequence keeps:
//                   w[i]   = exp(-exp(z[i] + w0[i]))                        (decay, float32)
//                   out[j] = sum_i r[i] (S[i][j] + u[i] k[i] v[j])
//                   S[i][j] = w[i] S[i][j] + k[i] v[j]
//                 and the last row's h goes into the state for the next pass's token shift
//   head norm     out[row, head] = o / sqrt(mean(o^2) + eps) * weight * silu(gate)
//
// The state of a sequence is one float32 array: heads x N x N, then `width` values of the last h.  State, decays
// and every sum are float32; r, k, v, the gate and h come in the activation type.  A sequence's result depends
// on its own rows and state only, and every sum runs in one fixed order, so it is the same bits however the
// sequence's tokens are cut into passes and whatever else is in a pass.
#include "common.cuh"

// ----------------------------------------------------------------------------------------
// token shift
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ mu, int n_mix, T* __restrict__ mixes,
                                       int64_t mix_stride, const float* __restrict__ state, int64_t state_stride,
                                       int64_t last_off, const int32_t* __restrict__ row_slot,
                                       const int32_t* __restrict__ row_pos, int n_rows, int width) {
    pdl_prologue();
    const int row = blockIdx.x;
    const int slot = row_slot[row], pos = row_pos[row];
    const bool above = row > 0 && slot >= 0 && row_slot[row - 1] == slot && row_pos[row - 1] == pos - 1;
    const T* cur = h + (int64_t)row * width;
    const T* prev_row = above ? cur - width : nullptr;
    const float* prev_state = (!above && slot >= 0) ? state + (int64_t)slot * state_stride + last_off : nullptr;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = to_f32(cur[c]);
        const float b = prev_row != nullptr ? to_f32(prev_row[c]) : (prev_state != nullptr ? prev_state[c] : 0.f);
        const float d = b - x;
        for (int s = 0; s < n_mix; ++s)
            mixes[(int64_t)s * mix_stride + (int64_t)row * width + c] = from_f32<T>(fmaf(d, mu[(int64_t)s * width + c], x));
    }
}

// ----------------------------------------------------------------------------------------
// scan: one block per (sequence, head); WKV_P threads share column j of S, each with NB / WKV_P of its N values in
// registers (key channels 4 (e WKV_P + p) + 0..3 for e = 0, 1, ...), so a token costs each thread NB / WKV_P steps of
// the recurrence, four partial sums that do not wait on each other, and two shuffles.  The rows of the next 16 tokens
// are fetched into registers while the current 16 are worked on out of shared memory.
// ----------------------------------------------------------------------------------------
#define WKV_TB 16      // tokens staged in shared memory at a time
#define WKV_P 4        // threads per column of the state

template <typename T, int NB>
__global__ void __launch_bounds__(NB * WKV_P) wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                                             const float* __restrict__ z, const float* __restrict__ w0,
                                                             const float* __restrict__ u, const T* __restrict__ h,
                                                             float* __restrict__ o, float* __restrict__ state, int64_t state_stride,
                                                             const int32_t* __restrict__ seq_first_row, const int32_t* __restrict__ seq_slot,
                                                             int heads, int N, int width) {
    constexpr int NT = NB * WKV_P;              // threads
    constexpr int PER = NB / WKV_P;             // state values per thread
    constexpr int FETCH = WKV_TB * NB / NT;     // values of each staged array a thread fetches per 16 tokens
    static_assert(PER % 4 == 0 && WKV_TB * NB % NT == 0, "the column split must leave groups of four key channels");
    __shared__ __align__(16) float rs[WKV_TB][NB], ks[WKV_TB][NB], ws[WKV_TB][NB], vs[WKV_TB][NB];
    __shared__ __align__(16) float us[NB], w0s[NB];
    pdl_launch_dependents();
    const int seq = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int j = tid / WKV_P, p = tid % WKV_P;
    const int64_t ld = (int64_t)heads * N;
    for (int i = tid; i < NB; i += NT) {
        us[i] = i < N ? u[head * N + i] : 0.f;
        w0s[i] = i < N ? w0[head * N + i] : 0.f;
    }
    pdl_wait();
    const int slot = seq_slot[seq];
    const int row0 = seq_first_row[seq], row1 = seq_first_row[seq + 1];
    if (slot < 0 || row1 <= row0) return;
    float* S = state + (int64_t)slot * state_stride + (int64_t)head * N * N;
    float s[PER];
#pragma unroll
    for (int e = 0; e < PER / 4; ++e)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int i = 4 * (e * WKV_P + p) + q;
            s[4 * e + q] = (i < N && j < N) ? S[(int64_t)i * N + j] : 0.f;
        }
    float fr[FETCH], fk[FETCH], fv[FETCH], fz[FETCH];
    auto fetch = [&](int t0) {
#pragma unroll
        for (int x = 0; x < FETCH; ++x) {
            const int e = tid + x * NT, t = e / NB, i = e % NB;
            const bool in = i < N && t0 + t < row1;
            const int64_t at = (int64_t)(t0 + t) * ld + (int64_t)head * N + i;
            fr[x] = in ? to_f32(r[at]) : 0.f;
            fk[x] = in ? to_f32(k[at]) : 0.f;
            fv[x] = in ? to_f32(v[at]) : 0.f;
            fz[x] = in ? z[at] : 0.f;
        }
    };
    fetch(row0);
    __syncthreads();                            // us, w0s
    for (int t0 = row0; t0 < row1; t0 += WKV_TB) {
        const int nt = min(WKV_TB, row1 - t0);
#pragma unroll
        for (int x = 0; x < FETCH; ++x) {
            const int e = tid + x * NT, t = e / NB, i = e % NB;
            rs[t][i] = fr[x];
            ks[t][i] = fk[x];
            vs[t][i] = fv[x];
            ws[t][i] = i < N ? expf(-expf(fz[x] + w0s[i])) : 0.f;
        }
        __syncthreads();
        if (t0 + WKV_TB < row1) fetch(t0 + WKV_TB);
        for (int t = 0; t < nt; ++t) {
            const float vj = vs[t][j];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < PER / 4; ++e) {
                const int i0 = 4 * (e * WKV_P + p);
                const float4 r4 = *reinterpret_cast<const float4*>(&rs[t][i0]);
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][i0]);
                const float4 w4 = *reinterpret_cast<const float4*>(&ws[t][i0]);
                const float4 u4 = *reinterpret_cast<const float4*>(&us[i0]);
                const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
                const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float kv = kk[q] * vj;
                    acc[q] = fmaf(rr[q], fmaf(uu[q], kv, s[4 * e + q]), acc[q]);
                    s[4 * e + q] = fmaf(ww[q], s[4 * e + q], kv);
                }
            }
            float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
            for (int off = 1; off < WKV_P; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (p == 0 && j < N) o[(int64_t)(t0 + t) * ld + (int64_t)head * N + j] = sum;
        }
        __syncthreads();
    }
#pragma unroll
    for (int e = 0; e < PER / 4; ++e)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int i = 4 * (e * WKV_P + p) + q;
            if (i < N && j < N) S[(int64_t)i * N + j] = s[4 * e + q];
        }
    if (head == 0) {        // the last row's h, for the token shift of the sequence's next token
        float* last = state + (int64_t)slot * state_stride + (int64_t)heads * N * N;
        const T* hr = h + (int64_t)(row1 - 1) * width;
        for (int c = tid; c < width; c += NT) last[c] = to_f32(hr[c]);
    }
}

// Any N: the state stays in global memory (read and written per token); thread j owns column j.
template <typename T>
__global__ void wkv_scan_any_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                    const float* __restrict__ z, const float* __restrict__ w0, const float* __restrict__ u,
                                    const T* __restrict__ h, float* __restrict__ o, float* __restrict__ state, int64_t state_stride,
                                    const int32_t* __restrict__ seq_first_row, const int32_t* __restrict__ seq_slot, int heads,
                                    int N, int width) {
    extern __shared__ float wk_smem[];       // r, k, w of the token: 3 N
    pdl_prologue();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int64_t ld = (int64_t)heads * N;
    const int slot = seq_slot[seq];
    const int row0 = seq_first_row[seq], row1 = seq_first_row[seq + 1];
    if (slot < 0 || row1 <= row0) return;
    float* S = state + (int64_t)slot * state_stride + (int64_t)head * N * N;
    float* rs = wk_smem;
    float* ks = rs + N;
    float* ws = ks + N;
    for (int t = row0; t < row1; ++t) {
        __syncthreads();
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            const int64_t at = (int64_t)t * ld + (int64_t)head * N + i;
            rs[i] = to_f32(r[at]);
            ks[i] = to_f32(k[at]);
            ws[i] = expf(-expf(z[at] + w0[head * N + i]));
        }
        __syncthreads();
        for (int j = threadIdx.x; j < N; j += blockDim.x) {
            const float vj = to_f32(v[(int64_t)t * ld + (int64_t)head * N + j]);
            float acc = 0.f;
            for (int i = 0; i < N; ++i) {
                const float kv = ks[i] * vj, sv = S[(int64_t)i * N + j];
                acc = fmaf(rs[i], fmaf(u[head * N + i], kv, sv), acc);
                S[(int64_t)i * N + j] = fmaf(ws[i], sv, kv);
            }
            o[(int64_t)t * ld + (int64_t)head * N + j] = acc;
        }
    }
    if (head == 0) {
        float* last = state + (int64_t)slot * state_stride + (int64_t)heads * N * N;
        const T* hr = h + (int64_t)(row1 - 1) * width;
        for (int c = threadIdx.x; c < width; c += blockDim.x) last[c] = to_f32(hr[c]);
    }
}

// ----------------------------------------------------------------------------------------
// head norm, weight and gate: one warp per (row, head)
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, const T* __restrict__ gate,
                                      T* __restrict__ out, int n_rows, int heads, int N, float eps) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_rows * heads) return;
    const int head = (int)(item % heads);
    const float* src = o + item * N;
    float ss = 0.f;
    for (int i = lane; i < N; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)N + eps);
    for (int i = lane; i < N; i += 32) {
        const float g = to_f32(gate[item * N + i]);
        out[item * N + i] = from_f32<T>(src[i] * scale * weight[head * N + i] * (g / (1.0f + expf(-g))));
    }
}

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------
X0NE_API int x0ne_token_shift_mix(const void* h, int dt, const float* mu, int n_mix, void* mixes, int64_t mix_stride, const float* state,
                                  int64_t state_stride, int64_t last_off, const int32_t* row_slot, const int32_t* row_pos,
                                  int n_rows, int width, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && width > 0 && n_mix > 0 && mix_stride >= (int64_t)n_rows * width && state_stride >= last_off + width,
                 "token_shift: rows %d width %d mixes %d", n_rows, width, n_mix);
    if (n_rows == 0) return 0;
    const int threads = width >= 256 ? 256 : (width + 31) / 32 * 32;
    if (dt == X0NE_F32)
        x0ne_launch(token_shift_mix_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)h, mu, n_mix, (float*)mixes, mix_stride, state, state_stride, last_off, row_slot, row_pos, n_rows, width);
    else if (dt == X0NE_BF16)
        x0ne_launch(token_shift_mix_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, (const bf16*)h, mu, n_mix, (bf16*)mixes, mix_stride, state, state_stride, last_off, row_slot, row_pos, n_rows, width);
    else
        X0NE_REQUIRE(false, "token_shift: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

template <typename T>
static int wkv_scan_launch(const T* r, const T* k, const T* v, const float* z, const float* w0, const float* u, const T* h, float* o,
                           float* state, int64_t state_stride, const int32_t* seq_first_row, const int32_t* seq_slot, int n_seqs,
                           int heads, int N, int width, cudaStream_t stream) {
    const dim3 grid(n_seqs, heads);
#define WKV_SCAN(NB) x0ne_launch(wkv_scan_kernel<T, NB>, grid, dim3(NB * WKV_P), 0, stream, r, k, v, z, w0, u, h, o, state, state_stride, seq_first_row, seq_slot, heads, N, width)
    if (N <= 32) WKV_SCAN(32);
    else if (N <= 64) WKV_SCAN(64);
    else if (N <= 96) WKV_SCAN(96);
    else if (N <= 128) WKV_SCAN(128);
    else {
        const int threads = N >= 256 ? 256 : (N + 31) / 32 * 32;
        x0ne_launch(wkv_scan_any_kernel<T>, grid, dim3(threads), (size_t)3 * N * sizeof(float), stream, r, k, v, z, w0, u, h, o, state, state_stride,
                    seq_first_row, seq_slot, heads, N, width);
    }
#undef WKV_SCAN
    X0NE_LAUNCH_CHECK();
}

// r, k, v: [rows][heads * N] in the activation type; z: float32 [rows][heads * N] (the decay's exponent before w0);
// h: [rows][width], the mixer's input; o: float32 [rows][heads * N]; state: float32 [slots][state_stride].
X0NE_API int x0ne_wkv_scan(const void* r, const void* k, const void* v, int dt, const float* z, const float* w0, const float* u,
                           const void* h, float* o, float* state, int64_t state_stride, const int32_t* seq_first_row,
                           const int32_t* seq_slot, int n_seqs, int heads, int N, int width, cudaStream_t stream) {
    X0NE_REQUIRE(n_seqs >= 0 && heads > 0 && heads <= 65535 && N > 0 && N <= 4096 && width > 0 && state_stride >= (int64_t)heads * N * N + width,
                 "wkv_scan: %d sequences, %d heads of %d, width %d", n_seqs, heads, N, width);
    if (n_seqs == 0) return 0;
    if (dt == X0NE_F32)
        return wkv_scan_launch<float>((const float*)r, (const float*)k, (const float*)v, z, w0, u, (const float*)h, o, state, state_stride, seq_first_row, seq_slot, n_seqs, heads, N, width, stream);
    if (dt == X0NE_BF16)
        return wkv_scan_launch<bf16>((const bf16*)r, (const bf16*)k, (const bf16*)v, z, w0, u, (const bf16*)h, o, state, state_stride, seq_first_row, seq_slot, n_seqs, heads, N, width, stream);
    X0NE_REQUIRE(false, "wkv_scan: unknown dtype tag %d", dt);
}

X0NE_API int x0ne_head_norm_gate(const float* o, const float* weight, const void* gate, void* out, int dt, int n_rows, int heads, int N,
                                 float eps, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && heads > 0 && N > 0, "head_norm_gate: rows %d heads %d of %d", n_rows, heads, N);
    if (n_rows == 0) return 0;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * heads;
    const unsigned grid = (unsigned)((items + warps - 1) / warps);
    if (dt == X0NE_F32)
        x0ne_launch(head_norm_gate_kernel<float>, dim3(grid), dim3(warps * 32), 0, stream, o, weight, (const float*)gate, (float*)out, n_rows, heads, N, eps);
    else if (dt == X0NE_BF16)
        x0ne_launch(head_norm_gate_kernel<bf16>, dim3(grid), dim3(warps * 32), 0, stream, o, weight, (const bf16*)gate, (bf16*)out, n_rows, heads, N, eps);
    else
        X0NE_REQUIRE(false, "head_norm_gate: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// out = tanh(x): float32 in, the activation type out (the inner activation of the decay's two small products)
template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ x, T* __restrict__ out, int64_t total) {
    pdl_prologue();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(tanhf(x[i]));
}

X0NE_API int x0ne_tanh_rows(const float* x, void* out, int dt, int64_t total, cudaStream_t stream) {
    X0NE_REQUIRE(total >= 0 && (dt == X0NE_F32 || dt == X0NE_BF16), "tanh: %lld values, dtype tag %d", (long long)total, dt);
    if (total == 0) return 0;
    const unsigned grid = (unsigned)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
    if (dt == X0NE_F32) x0ne_launch(tanh_rows_kernel<float>, dim3(grid), dim3(256), 0, stream, x, (float*)out, total);
    else x0ne_launch(tanh_rows_kernel<bf16>, dim3(grid), dim3(256), 0, stream, x, (bf16*)out, total);
    X0NE_LAUNCH_CHECK();
}
