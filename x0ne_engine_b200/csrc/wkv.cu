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

// 8 consecutive values as 16-byte accesses
__device__ __forceinline__ void wkv_load8(const bf16* p, float* v) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void wkv_load8(const float* p, float* v) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void wkv_store8(bf16* p, const float* v) {
    uint4 q;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = q;
}
__device__ __forceinline__ void wkv_store8(float* p, const float* v) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}

// The token shift with 8 values per thread (width, strides and offsets multiples of 8, 16-byte aligned bases):
// block (row, 8 x blockDim.x columns).
template <typename T>
__global__ void token_shift_mix_vec_kernel(const T* __restrict__ h, const float* __restrict__ mu, int n_mix, T* __restrict__ mixes,
                                           int64_t mix_stride, const float* __restrict__ state, int64_t state_stride,
                                           int64_t last_off, const int32_t* __restrict__ row_slot,
                                           const int32_t* __restrict__ row_pos, int n_rows, int width) {
    pdl_prologue();
    const int row = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    const int slot = row_slot[row], pos = row_pos[row];
    const bool above = row > 0 && slot >= 0 && row_slot[row - 1] == slot && row_pos[row - 1] == pos - 1;
    const T* cur = h + (int64_t)row * width + c;
    float x[8], b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    wkv_load8(cur, x);
    if (above) wkv_load8(cur - width, b);
    else if (slot >= 0) wkv_load8(state + (int64_t)slot * state_stride + last_off + c, b);
    for (int s = 0; s < n_mix; ++s) {
        float m[8], y[8];
        wkv_load8(mu + (int64_t)s * width + c, m);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = fmaf(b[i] - x[i], m[i], x[i]);
        wkv_store8(mixes + (int64_t)s * mix_stride + (int64_t)row * width + c, y);
    }
}

// ----------------------------------------------------------------------------------------
// scan.  The order of every sum is fixed and the same in both kernels below: out[j] is the sum over groups g of four
// key channels of  p_g = fma chain over the group's channels ascending (from 0),  and the p_g are added as a balanced
// tree (neighbours first).  So a token's result is the same bits whichever kernel ran it.
//
// wkv_scan_kernel (rows of many tokens): one block per (sequence, head, WKV_CB value columns of S); columns of S do
// not depend on one another, so a head is spread over blocks.  Two kinds of threads:
//   * 2 NB working threads: thread (g, jp) keeps the 4 x 2 tile of S at key channels 4 g .. 4 g + 3 and value columns
//     2 jp, 2 jp + 1 of the block in registers.  A token costs it four reads of shared memory (r, k, w of its four
//     channels, v of its two columns), 8 steps of the recurrence, one exchange with its neighbour in g (the first
//     level of the tree: one of the two goes on with the first column, the other with the second) and one store of
//     that sum to shared memory.  Only S is carried from token to token.
//   * WKV_PRODUCERS staging threads: they fetch r, k, v and the decay exponents two stages ahead into registers, work
//     out w = exp(-exp(z + w0)) and put all of it into the other half of a double buffer while the current half is
//     used; then they add the partial sums of the stage before (the tree's other levels) and write out.
// wkv_step_kernel (one token per sequence): one block per (sequence, head); thread (j, y) reads, uses and writes back
// the values of column j in its groups straight from and to the state, coalesced over j.
// ----------------------------------------------------------------------------------------
#define WKV_CB 16             // value columns of a block of the scan over many tokens
#define WKV_GI 4              // key channels of a group
#define WKV_PRODUCERS 128     // staging threads of a block

template <int G>
__device__ __forceinline__ float wkv_tree_sum(float (&q)[G]) {
#pragma unroll
    for (int w = 1; w < G; w <<= 1)
#pragma unroll
        for (int x = 0; x < G; x += 2 * w) q[x] += q[x + w];
    return q[0];
}

template <typename T, int NB>
__global__ void __launch_bounds__(2 * NB + WKV_PRODUCERS) wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                                                         const float* __restrict__ z, const float* __restrict__ w0,
                                                                         const float* __restrict__ u, const T* __restrict__ h,
                                                                         float* __restrict__ o, float* __restrict__ state, int64_t state_stride,
                                                                         const int32_t* __restrict__ seq_first_row, const int32_t* __restrict__ seq_slot,
                                                                         int heads, int N, int width) {
    constexpr int G = NB / WKV_GI;                  // groups of key channels = working threads that share a column
    constexpr int H = G / 2;                        // partial sums of a column that reach shared memory
    constexpr int NC = G * (WKV_CB / 2);            // working threads: 2 NB
    constexpr int TB = NB <= 64 ? 16 : 8;           // tokens staged at a time
    constexpr int PER = TB * NB / WKV_PRODUCERS;    // values of r, k, z a staging thread fetches per stage
    constexpr int PV = TB * WKV_CB / WKV_PRODUCERS; // values of v, and results it adds up
    constexpr int TSTEP = WKV_PRODUCERS / NB;
    static_assert(H >= 4 && (G & (G - 1)) == 0 && G <= 32 && WKV_PRODUCERS % NB == 0 && PER >= 1 && PV >= 1 && NC == 2 * NB, "tile shape");
    __shared__ __align__(16) float rs[2][TB][NB], ks[2][TB][NB], ws[2][TB][NB], vs[2][TB][WKV_CB];
    __shared__ __align__(16) float part[2][TB][WKV_CB][H];
    pdl_launch_dependents();
    const int seq = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * WKV_CB, tid = threadIdx.x;
    const int64_t ld = (int64_t)heads * N;
    const bool producer = tid >= NC;
    const int pt = tid - NC, pi = pt % NB, ptb = pt / NB;           // staging: its key channel and first token
    const int g = tid % G, jc = 2 * ((tid / G) % (WKV_CB / 2)), i0 = WKV_GI * g;      // working: its tile
    float w0r = 0.f, ur[WKV_GI];
#pragma unroll
    for (int a = 0; a < WKV_GI; ++a) ur[a] = 0.f;
    if (producer) {
        if (pi < N) w0r = w0[head * N + pi];
    } else {
#pragma unroll
        for (int a = 0; a < WKV_GI; ++a)
            if (i0 + a < N) ur[a] = u[head * N + i0 + a];
    }
    pdl_wait();
    const int slot = seq_slot[seq];
    const int row0 = seq_first_row[seq], row1 = seq_first_row[seq + 1];
    if (slot < 0 || row1 <= row0 || j0 >= N) return;
    float* S = state + (int64_t)slot * state_stride + (int64_t)head * N * N;
    const int n_stages = (row1 - row0 + TB - 1) / TB;

    float fr[PER], fk[PER], fz[PER], fv[PV];            // a staging thread's share of one stage, on its way
    auto fetch = [&](int at_stage) {
        const int t0 = row0 + at_stage * TB;
#pragma unroll
        for (int x = 0; x < PER; ++x) {
            // every fetch is made, from an address inside the sequence's rows, so that none waits for another;
            // rows past the sequence's last are not used, channels past the head's last are zeroed in `put`
            const int64_t at = (int64_t)min(t0 + ptb + x * TSTEP, row1 - 1) * ld + (int64_t)head * N + min(pi, N - 1);
            fr[x] = to_f32(r[at]);
            fk[x] = to_f32(k[at]);
            fz[x] = z[at];
        }
#pragma unroll
        for (int x = 0; x < PV; ++x) {
            const int e = pt + x * WKV_PRODUCERS, t = e / WKV_CB, c = e % WKV_CB;
            fv[x] = to_f32(v[(int64_t)min(t0 + t, row1 - 1) * ld + (int64_t)head * N + min(j0 + c, N - 1)]);
        }
    };
    auto put = [&](int buf) {
#pragma unroll
        for (int x = 0; x < PER; ++x) {
            const int t = ptb + x * TSTEP;
            rs[buf][t][pi] = pi < N ? fr[x] : 0.f;
            ks[buf][t][pi] = pi < N ? fk[x] : 0.f;
            ws[buf][t][pi] = pi < N ? expf(-expf(fz[x] + w0r)) : 0.f;
        }
#pragma unroll
        for (int x = 0; x < PV; ++x) {
            const int e = pt + x * WKV_PRODUCERS, c = e % WKV_CB;
            vs[buf][e / WKV_CB][c] = j0 + c < N ? fv[x] : 0.f;
        }
    };
    auto write_out = [&](int at_stage, int buf) {       // the results of a stage the working threads are done with
        const int t0 = row0 + at_stage * TB;
#pragma unroll
        for (int x = 0; x < PV; ++x) {
            const int e = pt + x * WKV_PRODUCERS, t = e / WKV_CB, c = e % WKV_CB;
            if (t0 + t >= row1 || j0 + c >= N) continue;
            float q[H];
#pragma unroll
            for (int y = 0; y < H; y += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(&part[buf][t][c][y]);
                q[y] = q4.x; q[y + 1] = q4.y; q[y + 2] = q4.z; q[y + 3] = q4.w;
            }
            o[(int64_t)(t0 + t) * ld + (int64_t)head * N + j0 + c] = wkv_tree_sum<H>(q);
        }
    };

    float s[WKV_GI][2];
    if (producer) {
        fetch(0);
        put(0);
        if (n_stages > 1) fetch(1);
    } else {
#pragma unroll
        for (int a = 0; a < WKV_GI; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
                s[a][b] = (i0 + a < N && j0 + jc + b < N) ? S[(int64_t)(i0 + a) * N + j0 + jc + b] : 0.f;
    }
    __syncthreads();
    for (int it = 0; it < n_stages; ++it) {
        const int buf = it & 1;
        if (producer) {
            if (it + 1 < n_stages) put(buf ^ 1);            // fetched a whole stage ago
            if (it + 2 < n_stages) fetch(it + 2);
            if (it > 0) write_out(it - 1, buf ^ 1);
        } else {
            const int nt = min(TB, row1 - (row0 + it * TB));
            const bool odd = (g & 1) != 0;
            float* mine = &part[buf][0][jc + (odd ? 1 : 0)][g >> 1];
#pragma unroll 4
            for (int t = 0; t < nt; ++t) {
                const float4 r4 = *reinterpret_cast<const float4*>(&rs[buf][t][i0]);
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[buf][t][i0]);
                const float4 w4 = *reinterpret_cast<const float4*>(&ws[buf][t][i0]);
                const float2 v2 = *reinterpret_cast<const float2*>(&vs[buf][t][jc]);
                const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
                const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, vv[2] = {v2.x, v2.y};
                float acc[2] = {0.f, 0.f};
#pragma unroll
                for (int a = 0; a < WKV_GI; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const float kv = kk[a] * vv[b];
                        acc[b] = fmaf(rr[a], fmaf(ur[a], kv, s[a][b]), acc[b]);
                        s[a][b] = fmaf(ww[a], s[a][b], kv);
                    }
                // groups g and g ^ 1: the even one goes on with the first column's sum, the odd one with the second's
                const float sum = (odd ? acc[1] : acc[0]) + __shfl_xor_sync(0xffffffffu, odd ? acc[0] : acc[1], 1);
                mine[t * (WKV_CB * H)] = sum;
            }
        }
        __syncthreads();
    }
    if (producer) {
        write_out(n_stages - 1, (n_stages - 1) & 1);
    } else {
#pragma unroll
        for (int a = 0; a < WKV_GI; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
                if (i0 + a < N && j0 + jc + b < N) S[(int64_t)(i0 + a) * N + j0 + jc + b] = s[a][b];
    }
    if (head == 0 && blockIdx.z == 0) {        // the last row's h, for the token shift of the sequence's next token
        float* last = state + (int64_t)slot * state_stride + (int64_t)heads * N * N;
        const T* hr = h + (int64_t)(row1 - 1) * width;
        for (int c = tid; c < width; c += NC + WKV_PRODUCERS) last[c] = to_f32(hr[c]);
    }
}

// One token per sequence (more are worked through one after the other): block (NB, GY); thread (j, y) takes the groups
// y, y + GY, ... of column j.
template <typename T, int NB, int GY>
__global__ void __launch_bounds__(NB * GY) wkv_step_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                                          const float* __restrict__ z, const float* __restrict__ w0,
                                                          const float* __restrict__ u, const T* __restrict__ h,
                                                          float* __restrict__ o, float* __restrict__ state, int64_t state_stride,
                                                          const int32_t* __restrict__ seq_first_row, const int32_t* __restrict__ seq_slot,
                                                          int heads, int N, int width) {
    constexpr int G = NB / WKV_GI;
    __shared__ __align__(16) float rs[NB], ks[NB], ws[NB], us[NB], w0s[NB];
    __shared__ float part[G][NB];
    pdl_launch_dependents();
    const int seq = blockIdx.x, head = blockIdx.y, j = threadIdx.x, y0 = threadIdx.y, tid = threadIdx.y * NB + threadIdx.x;
    const int64_t ld = (int64_t)heads * N;
    if (tid < NB) {
        us[tid] = tid < N ? u[head * N + tid] : 0.f;
        w0s[tid] = tid < N ? w0[head * N + tid] : 0.f;
    }
    pdl_wait();
    const int slot = seq_slot[seq];
    const int row0 = seq_first_row[seq], row1 = seq_first_row[seq + 1];
    if (slot < 0 || row1 <= row0) return;
    float* S = state + (int64_t)slot * state_stride + (int64_t)head * N * N;
    for (int t = row0; t < row1; ++t) {
        __syncthreads();
        if (tid < NB) {
            const int64_t at = (int64_t)t * ld + (int64_t)head * N + tid;
            const bool in = tid < N;
            rs[tid] = in ? to_f32(r[at]) : 0.f;
            ks[tid] = in ? to_f32(k[at]) : 0.f;
            ws[tid] = in ? expf(-expf(z[at] + w0s[tid])) : 0.f;
        }
        const float vj = j < N ? to_f32(v[(int64_t)t * ld + (int64_t)head * N + j]) : 0.f;
        float sv[(G + GY - 1) / GY][WKV_GI];
#pragma unroll
        for (int x = 0; x < (G + GY - 1) / GY; ++x) {
            const int g = y0 + x * GY;
#pragma unroll
            for (int a = 0; a < WKV_GI; ++a) {
                const int i = WKV_GI * g + a;
                sv[x][a] = (g < G && i < N && j < N) ? S[(int64_t)i * N + j] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int x = 0; x < (G + GY - 1) / GY; ++x) {
            const int g = y0 + x * GY;
            if (g >= G) continue;
            float acc = 0.f;
#pragma unroll
            for (int a = 0; a < WKV_GI; ++a) {
                const int i = WKV_GI * g + a;
                const float kv = ks[i] * vj;
                acc = fmaf(rs[i], fmaf(us[i], kv, sv[x][a]), acc);
                if (i < N && j < N) S[(int64_t)i * N + j] = fmaf(ws[i], sv[x][a], kv);
            }
            part[g][j] = acc;
        }
        __syncthreads();
        if (y0 == 0 && j < N) {
            float q[G];
#pragma unroll
            for (int x = 0; x < G; ++x) q[x] = part[x][j];
            o[(int64_t)t * ld + (int64_t)head * N + j] = wkv_tree_sum<G>(q);
        }
    }
    if (head == 0) {
        float* last = state + (int64_t)slot * state_stride + (int64_t)heads * N * N;
        const T* hr = h + (int64_t)(row1 - 1) * width;
        for (int c = tid; c < width; c += NB * GY) last[c] = to_f32(hr[c]);
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

// The same with 8 values per lane: LANES = N / 8 lanes (a power of two up to 32) work on one (row, head).
template <typename T, int LANES>
__global__ void head_norm_gate_vec_kernel(const float* __restrict__ o, const float* __restrict__ weight, const T* __restrict__ gate,
                                          T* __restrict__ out, int64_t items, int heads, float eps) {
    pdl_prologue();
    constexpr int N = LANES * 8;
    const int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LANES;
    const int part = threadIdx.x % LANES;
    const bool live = item < items;
    const int64_t at = (live ? item : 0) * N + part * 8;
    float x[8], g[8], w[8], y[8];
    wkv_load8(o + at, x);
    wkv_load8(gate + at, g);
    wkv_load8(weight + (int)((live ? item : 0) % heads) * N + part * 8, w);
    // the order of the scalar kernel's sum is not kept: the result is the same to rounding
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
#pragma unroll
    for (int off = LANES / 2; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float scale = 1.0f / sqrtf(ss / (float)N + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = x[i] * scale * w[i] * (g[i] / (1.0f + expf(-g[i])));
    if (live) wkv_store8(out + at, y);
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
    if ((dt == X0NE_F32 || dt == X0NE_BF16) && width % 8 == 0 && mix_stride % 8 == 0 && state_stride % 4 == 0 && last_off % 4 == 0 &&
        ((((uintptr_t)h | (uintptr_t)mu | (uintptr_t)mixes | (uintptr_t)state) & 15) == 0)) {
        const int vthreads = width / 8 >= 128 ? 128 : (width / 8 + 31) / 32 * 32;
        const dim3 vgrid(n_rows, (width / 8 + vthreads - 1) / vthreads);
        if (dt == X0NE_F32)
            x0ne_launch(token_shift_mix_vec_kernel<float>, vgrid, dim3(vthreads), 0, stream, (const float*)h, mu, n_mix, (float*)mixes, mix_stride, state, state_stride, last_off, row_slot, row_pos, n_rows, width);
        else
            x0ne_launch(token_shift_mix_vec_kernel<bf16>, vgrid, dim3(vthreads), 0, stream, (const bf16*)h, mu, n_mix, (bf16*)mixes, mix_stride, state, state_stride, last_off, row_slot, row_pos, n_rows, width);
        X0NE_LAUNCH_CHECK();
    }
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
                           int heads, int N, int width, int one_token, cudaStream_t stream) {
    const dim3 grid(n_seqs, heads);
#define WKV_ARGS r, k, v, z, w0, u, h, o, state, state_stride, seq_first_row, seq_slot, heads, N, width
#define WKV_SCAN(NB) x0ne_launch(wkv_scan_kernel<T, NB>, dim3(n_seqs, heads, NB / WKV_CB), dim3(2 * NB + WKV_PRODUCERS), 0, stream, WKV_ARGS)
#define WKV_STEP(NB, GY) x0ne_launch(wkv_step_kernel<T, NB, GY>, grid, dim3(NB, GY), 0, stream, WKV_ARGS)
    if (N <= 32) { if (one_token) WKV_STEP(32, 4); else WKV_SCAN(32); }
    else if (N <= 64) { if (one_token) WKV_STEP(64, 8); else WKV_SCAN(64); }
    else if (N <= 128) { if (one_token) WKV_STEP(128, 4); else WKV_SCAN(128); }
    else {
        const int threads = N >= 256 ? 256 : (N + 31) / 32 * 32;
        x0ne_launch(wkv_scan_any_kernel<T>, grid, dim3(threads), (size_t)3 * N * sizeof(float), stream, WKV_ARGS);
    }
#undef WKV_SCAN
#undef WKV_STEP
#undef WKV_ARGS
    X0NE_LAUNCH_CHECK();
}

// r, k, v: [rows][heads * N] in the activation type; z: float32 [rows][heads * N] (the decay's exponent before w0);
// h: [rows][width], the mixer's input; o: float32 [rows][heads * N]; state: float32 [slots][state_stride].
// one_token != 0 says that every sequence brings one row (the kernel made for that runs; it is right for any number).
X0NE_API int x0ne_wkv_scan(const void* r, const void* k, const void* v, int dt, const float* z, const float* w0, const float* u,
                           const void* h, float* o, float* state, int64_t state_stride, const int32_t* seq_first_row,
                           const int32_t* seq_slot, int n_seqs, int heads, int N, int width, int one_token, cudaStream_t stream) {
    X0NE_REQUIRE(n_seqs >= 0 && heads > 0 && heads <= 65535 && N > 0 && N <= 4096 && width > 0 && state_stride >= (int64_t)heads * N * N + width,
                 "wkv_scan: %d sequences, %d heads of %d, width %d", n_seqs, heads, N, width);
    if (n_seqs == 0) return 0;
    if (dt == X0NE_F32)
        return wkv_scan_launch<float>((const float*)r, (const float*)k, (const float*)v, z, w0, u, (const float*)h, o, state, state_stride, seq_first_row, seq_slot, n_seqs, heads, N, width, one_token, stream);
    if (dt == X0NE_BF16)
        return wkv_scan_launch<bf16>((const bf16*)r, (const bf16*)k, (const bf16*)v, z, w0, u, (const bf16*)h, o, state, state_stride, seq_first_row, seq_slot, n_seqs, heads, N, width, one_token, stream);
    X0NE_REQUIRE(false, "wkv_scan: unknown dtype tag %d", dt);
}

X0NE_API int x0ne_head_norm_gate(const float* o, const float* weight, const void* gate, void* out, int dt, int n_rows, int heads, int N,
                                 float eps, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && heads > 0 && N > 0, "head_norm_gate: rows %d heads %d of %d", n_rows, heads, N);
    if (n_rows == 0) return 0;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * heads;
    const int lanes = N / 8;
    if ((dt == X0NE_F32 || dt == X0NE_BF16) && N % 8 == 0 && (lanes & (lanes - 1)) == 0 && lanes <= 32 &&
        ((((uintptr_t)o | (uintptr_t)weight | (uintptr_t)gate | (uintptr_t)out) & 15) == 0)) {
        const int per_block = 128 / lanes;
        const dim3 vgrid((unsigned)((items + per_block - 1) / per_block));
#define HNG(L)                                                                                                                        \
        if (dt == X0NE_F32) x0ne_launch(head_norm_gate_vec_kernel<float, L>, vgrid, dim3(128), 0, stream, o, weight, (const float*)gate, (float*)out, items, heads, eps); \
        else x0ne_launch(head_norm_gate_vec_kernel<bf16, L>, vgrid, dim3(128), 0, stream, o, weight, (const bf16*)gate, (bf16*)out, items, heads, eps)
        switch (lanes) {
            case 1: HNG(1); break;
            case 2: HNG(2); break;
            case 4: HNG(4); break;
            case 8: HNG(8); break;
            case 16: HNG(16); break;
            default: HNG(32); break;
        }
#undef HNG
        X0NE_LAUNCH_CHECK();
    }
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
