// Routed feed-forward (mixture of experts): the router's choice, the grouping of (row, choice) pairs by
// expert, the experts' two products over the grouped pairs, and the weighted sum.
//
//   scores   s = softmax(z) over all router outputs, float32
//   choice   c = s + correction; outputs form `groups` equal groups of neighbours, a group's value is
//            its largest c, only the `keep` best groups stay (the others' c count as minus infinity);
//            the `top` largest c are chosen (equal values: the lower index first)
//   weights  the chosen outputs' s, as they are
// or, for a router that chooses on its logits (`on_logits`): s = z + correction (a bias of the router) without a
// softmax, the `top` largest s are chosen, and the weights are the softmax over the chosen s alone.
// A third kind of router (`mode` 2) scores with s = sigmoid(z) (+ correction for the choice, if there is one).  For every kind a
// group may be worth the sum of its `group_top` largest values instead of its largest one, and the chosen weights may
// be divided by their sum (+ 1e-20) and multiplied by a constant (`normalize`, `weight_scale`).
// The last `n - experts` router outputs are identity experts: their output is the row itself, they
// have no weights and form no group of pairs.
//
// A pair is (row, j-th choice), numbered row * top + j.  Pairs of one expert are listed together; the
// two products run over tiles of one expert's pairs, so an expert's weights are read once per tile of
// its pairs.  Every output value is one chain of fused multiply-adds over k in ascending order
// (float32), or one accumulator of the tensor-core tiles (bfloat16): it does not depend on where in
// the list a pair lies, so a row's result does not depend on what else is in the pass.
//
// Everything a launch's grid depends on is known on the host (rows, top, experts, widths): the tile
// table is sized for the worst case and unused tiles return at once, so the launches can be replayed
// from a CUDA graph.
#include "common.cuh"

#define MOE_TILE_M 32     // pairs per tile of the grouped products (all kernels of this library agree on it)

// ----------------------------------------------------------------------------------------
// Router: one warp per row.  z [rows][ldz] float32 (the router's n outputs first; the shared
// expert's gate logit at column sg_col when sgate is given).
// ----------------------------------------------------------------------------------------
__global__ void moe_route_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ correction, int n, int groups,
                                 int keep, int top, int n_rows, int32_t* __restrict__ chosen, float* __restrict__ weights,
                                 float* __restrict__ sgate, int sg_col, int mode, int group_top, int normalize, float weight_scale) {
    extern __shared__ float rt_smem[];
    pdl_prologue();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int row = blockIdx.x * warps + w;
    if (row >= n_rows) return;
    float* s = rt_smem + (size_t)w * (2 * n + groups);     // scores
    float* c = s + n;                                       // choice values
    float* gv = c + n;                                      // group values
    const float* zr = z + (int64_t)row * ldz;
    const bool on_logits = mode == 1;
    if (on_logits) {
        for (int i = lane; i < n; i += 32) {
            s[i] = zr[i] + correction[i];
            c[i] = s[i];
        }
    } else if (mode == 2) {
        for (int i = lane; i < n; i += 32) {
            s[i] = 1.0f / (1.0f + expf(-zr[i]));
            c[i] = correction != nullptr ? s[i] + correction[i] : s[i];
        }
    } else {
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, zr[i]);
        m = warp_max(m);
        float sum = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float e = expf(zr[i] - m);
            s[i] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        for (int i = lane; i < n; i += 32) {
            s[i] = s[i] / sum;
            c[i] = s[i] + correction[i];
        }
    }
    __syncwarp();
    const int per = n / groups;
    if (groups > 1 && keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            if (group_top <= 1) {
                for (int i = 0; i < per; ++i) b = fmaxf(b, c[g * per + i]);
            } else {
                // the sum of the group's `group_top` largest values, taken one after the other (a value taken is passed over
                // by its index, so equal values count as often as they occur)
                float sum = 0.f, last = INFINITY;
                int last_i = -1;
                for (int r = 0; r < group_top && r < per; ++r) {
                    float bv = -INFINITY;
                    int bi = -1;
                    for (int i = 0; i < per; ++i) {
                        const float v = c[g * per + i];
                        const bool open = v < last || (v == last && i > last_i);
                        if (open && (v > bv || bi < 0)) { bv = v; bi = i; }
                    }
                    if (bi < 0) break;
                    sum += bv;
                    last = bv;
                    last_i = bi;
                }
                b = sum;
            }
            gv[g] = b;
        }
        __syncwarp();
        // the `keep` best groups, one at a time (largest value, lowest index among equals); a kept group is
        // marked by +inf in gv, and afterwards every group that is not marked loses its experts
        for (int r = 0; r < keep; ++r) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gv[g];
                if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0 && bi != 0x7fffffff) gv[bi] = INFINITY;
            __syncwarp();
        }
        for (int i = lane; i < n; i += 32)
            if (gv[i / per] != INFINITY) c[i] = -INFINITY;
        __syncwarp();
    }
    for (int r = 0; r < top; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float v = c[i];
            if (v != INFINITY && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;        // (fewer allowed outputs than `top`, or a row of NaN: the first output, its own score)
        if (lane == 0) {
            chosen[(int64_t)row * top + r] = bi;
            weights[(int64_t)row * top + r] = s[bi];
            c[bi] = INFINITY;                // taken
        }
        __syncwarp();
    }
    if (on_logits && lane == 0) {       // softmax over the chosen values, in the order they were chosen (the first is the largest)
        float* wr = weights + (int64_t)row * top;
        const float m = wr[0];
        float sum = 0.f;
        for (int r = 0; r < top; ++r) {
            wr[r] = expf(wr[r] - m);
            sum += wr[r];
        }
        for (int r = 0; r < top; ++r) wr[r] = wr[r] / sum;
    }
    if (normalize && lane == 0) {       // the chosen scores over their sum, times the router's scale, in the order they were chosen
        float* wr = weights + (int64_t)row * top;
        float sum = 0.f;
        for (int r = 0; r < top; ++r) sum += wr[r];
        for (int r = 0; r < top; ++r) wr[r] = wr[r] / (sum + 1e-20f) * weight_scale;
    }
    if (sgate != nullptr && lane == 0) sgate[row] = 1.0f / (1.0f + expf(-zr[sg_col]));
}

// ----------------------------------------------------------------------------------------
// Grouping: pairs listed expert by expert, and the table of tiles.  One block.
//   offsets [experts + 1]   first place of each expert in `listed`
//   listed  [pairs]         pair numbers, expert by expert (identity choices are in no list)
//   tiles   [max_tiles][3]  expert, first place, count (count 0: the tile does not exist); tiles of tile_m pairs
//   n_tiles_out             how many tiles exist (optional)
// ----------------------------------------------------------------------------------------
__global__ void moe_group_kernel(const int32_t* __restrict__ chosen, int pairs, int experts, int32_t* __restrict__ offsets,
                                 int32_t* __restrict__ listed, int32_t* __restrict__ tiles, int max_tiles, int tile_m,
                                 int32_t* __restrict__ n_tiles_out) {
    extern __shared__ int gp_smem[];
    int* count = gp_smem;                 // [experts]
    int* start = count + experts;         // [experts + 1]
    int* tile0 = start + experts + 1;     // [experts + 1]
    pdl_prologue();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, t = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = at;
            tile0[e] = t;
            at += count[e];
            t += (count[e] + tile_m - 1) / tile_m;
        }
        start[experts] = at;
        tile0[experts] = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int n = count[e];
        for (int i = 0, t = tile0[e]; i < n && t < max_tiles; i += tile_m, ++t) {
            tiles[3 * t] = e;
            tiles[3 * t + 1] = start[e] + i;
            tiles[3 * t + 2] = min(tile_m, n - i);
        }
    }
    for (int t = tile0[experts] + threadIdx.x; t < max_tiles; t += blockDim.x) tiles[3 * t + 2] = 0;
    if (threadIdx.x == 0 && n_tiles_out != nullptr) n_tiles_out[0] = min(tile0[experts], max_tiles);
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) listed[start[e] + atomicAdd(&count[e], 1)] = p;
    }
}

// ----------------------------------------------------------------------------------------
// The experts' products over the tiles, on the CUDA cores: one fused multiply-add chain per output
// over k ascending (the 32-bit path; also the path of shapes the tensor-core kernel does not take).
//   ACT 1 (up):       act[pair][n] = relu(sum_k x[pair / top][k] w[e][n][k])^2             (activation type)
//   ACT 2 (gated up): act[pair][n] = silu(sum_k x[..][k] w[e][n][k]) * sum_k x[..][k] w[e][N + n][k]
//                     (an expert's weight holds its N gate rows, then its N up rows)
//   ACT 0 (down):     y[pair][n]   = sum_k act[pair][k] w[e][n][k]                          (float32)
// Tile 32 pairs x 64 outputs x 16 k, 256 threads, 2 x 4 outputs per thread.
// ----------------------------------------------------------------------------------------
template <typename T, int ACT>
__global__ void __launch_bounds__(256) moe_product_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ w, int N, int K,
                                                          const int32_t* __restrict__ listed, const int32_t* __restrict__ tiles,
                                                          int top, void* __restrict__ out, int pair_block) {
    __shared__ float As[16][MOE_TILE_M + 4];
    __shared__ float Ws[16][64 + 4];
    __shared__ float Us[ACT == 2 ? 16 : 1][64 + 4];
    __shared__ int pair_s[MOE_TILE_M];
    constexpr bool UP = ACT != 0;
    pdl_prologue();
    const int tile = blockIdx.y;
    const int count = tiles[3 * tile + 2];
    if (count <= 0) return;
    const int e = tiles[3 * tile], first = tiles[3 * tile + 1];
    const int tid = threadIdx.x, n0 = blockIdx.x * 64;
    if (tid < MOE_TILE_M) pair_s[tid] = tid < count ? listed[first + tid] : -1;
    __syncthreads();
    const T* we = w + (int64_t)e * (ACT == 2 ? 2 : 1) * N * K;
    const int tx = tid % 16, ty = tid / 16;
    float acc[2][4] = {};
    float acu[ACT == 2 ? 2 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = tid + it * 256;
            const int r = idx / 16, kk = idx % 16;
            const int p = pair_s[r], gk = k0 + kk;
            As[kk][r] = (p >= 0 && gk < K) ? to_f32(a[(int64_t)(UP ? p / top : p) * lda + gk]) : 0.f;
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int r = idx / 16, kk = idx % 16;
            const int gn = n0 + r, gk = k0 + kk;
            if (ACT == 2) {
                // gate row gn and its up row: all gate rows then all up rows, or blocks of pair_block gate rows and their up rows
                const int64_t gr = pair_block > 0 ? (int64_t)(gn / pair_block) * 2 * pair_block + gn % pair_block : gn;
                const int64_t ur = gr + (pair_block > 0 ? pair_block : N);
                Ws[kk][r] = (gn < N && gk < K) ? to_f32(we[gr * K + gk]) : 0.f;
                Us[kk][r] = (gn < N && gk < K) ? to_f32(we[ur * K + gk]) : 0.f;
            } else {
                Ws[kk][r] = (gn < N && gk < K) ? to_f32(we[(int64_t)gn * K + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float av[2], bv[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) av[i] = As[kk][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            if (ACT == 2) {
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acu[i][j] = fmaf(av[i], Us[kk][tx * 4 + j], acu[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = pair_s[ty * 2 + i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            if (ACT == 2) {
                const float g = acc[i][j];
                ((T*)out)[(int64_t)p * N + gn] = from_f32<T>(g / (1.0f + expf(-g)) * acu[i][j]);
            } else if (UP) {
                const float r = fmaxf(acc[i][j], 0.f);
                ((T*)out)[(int64_t)p * N + gn] = from_f32<T>(r * r);
            } else {
                ((float*)out)[(int64_t)p * N + gn] = acc[i][j];
            }
        }
    }
}

// ----------------------------------------------------------------------------------------
// Weighted sum: out[row] = sum_j weight_j (y[row * top + j] | x[row] for an identity choice)
//                          + sgate[row] * shared[row], in float32, choices in order.  One block per row.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ x, const int32_t* __restrict__ chosen,
                                   const float* __restrict__ weights, int top, int experts, const T* __restrict__ shared,
                                   const float* __restrict__ sgate, T* __restrict__ out, int hidden) {
    pdl_prologue();
    const int row = blockIdx.x;
    const int32_t* ch = chosen + (int64_t)row * top;
    const float* wt = weights + (int64_t)row * top;
    const float sg = shared != nullptr ? (sgate != nullptr ? sgate[row] : 1.f) : 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = ch[j];
            const float v = e < experts ? y[((int64_t)row * top + j) * hidden + c] : to_f32(x[(int64_t)row * hidden + c]);
            acc = fmaf(wt[j], v, acc);
        }
        if (shared != nullptr) acc = fmaf(sg, to_f32(shared[(int64_t)row * hidden + c]), acc);
        out[(int64_t)row * hidden + c] = from_f32<T>(acc);
    }
}

// The same four columns per thread with 16-byte reads of y (hidden % 4 == 0, aligned rows): grid (column blocks, rows).
__device__ __forceinline__ void cmb_load4(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void cmb_load4(const bf16* p, float* v) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void cmb_store4(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void cmb_store4(bf16* p, const float* v) {
    uint2 u;
    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
}
#define CMB_MAX_TOP 16
template <typename T>
__global__ void moe_combine_vec_kernel(const float* __restrict__ y, const T* __restrict__ x, const int32_t* __restrict__ chosen,
                                       const float* __restrict__ weights, int top, int experts, const T* __restrict__ shared,
                                       const float* __restrict__ sgate, T* __restrict__ out, int hidden) {
    pdl_prologue();
    const int row = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= hidden) return;
    const int32_t* ch = chosen + (int64_t)row * top;
    const float* wt = weights + (int64_t)row * top;
    float v[CMB_MAX_TOP][4], g[CMB_MAX_TOP];
    float xs[4], sv[4] = {0.f, 0.f, 0.f, 0.f};
    cmb_load4(x + (int64_t)row * hidden + c, xs);
#pragma unroll
    for (int j = 0; j < CMB_MAX_TOP; ++j) {
        if (j < top) {
            g[j] = wt[j];
            if (ch[j] < experts) cmb_load4(y + ((int64_t)row * top + j) * hidden + c, v[j]);      // (all the loads are in flight together)
            else { v[j][0] = xs[0]; v[j][1] = xs[1]; v[j][2] = xs[2]; v[j][3] = xs[3]; }
        }
    }
    const float sg = shared != nullptr ? (sgate != nullptr ? sgate[row] : 1.f) : 0.f;
    if (shared != nullptr) cmb_load4(shared + (int64_t)row * hidden + c, sv);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < CMB_MAX_TOP; ++j)
        if (j < top) {
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[k] = fmaf(g[j], v[j][k], acc[k]);
        }
    if (shared != nullptr) {
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = fmaf(sg, sv[k], acc[k]);
    }
    cmb_store4(out + (int64_t)row * hidden + c, acc);
}

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------
X0NE_API int x0ne_moe_tile_rows() { return MOE_TILE_M; }

// Tiles of tile_m pairs a pass of `pairs` pairs over `experts` experts can need at most.
X0NE_API int x0ne_moe_max_tiles(int pairs, int experts, int tile_m) {
    const int full = pairs / tile_m + experts;              // every expert may end in a partial tile
    return full < pairs ? full : (pairs > 0 ? pairs : 1);   // (never more tiles than pairs)
}

X0NE_API int x0ne_moe_route(const float* z, int ldz, const float* correction, int n, int groups, int keep, int top, int n_rows,
                            int32_t* chosen, float* weights, float* sgate, int sg_col, int mode, int group_top, int normalize,
                            float weight_scale, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && n > 0 && ldz >= n && top > 0 && top <= n, "moe_route: rows %d outputs %d ld %d top %d", n_rows, n, ldz, top);
    X0NE_REQUIRE(mode >= 0 && mode <= 2 && group_top >= 1 && (correction != nullptr || mode == 2), "moe_route: mode %d, group worth of %d values", mode, group_top);
    X0NE_REQUIRE(groups >= 1 && n % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (n / groups),
                 "moe_route: %d outputs in %d groups of which %d stay cannot give %d choices", n, groups, keep, top);
    X0NE_REQUIRE(sgate == nullptr || (sg_col >= n && sg_col < ldz), "moe_route: the shared gate's column %d lies outside the rows", sg_col);
    if (n_rows == 0) return 0;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * n + groups) * sizeof(float);
    X0NE_REQUIRE(smem <= 48 * 1024, "moe_route: %d router outputs are more than the kernel holds", n);
    x0ne_launch(moe_route_kernel, dim3((n_rows + warps - 1) / warps), dim3(warps * 32), smem, stream, z, ldz, correction, n, groups, keep,
                top, n_rows, chosen, weights, sgate, sg_col, mode, group_top, normalize, weight_scale);
    X0NE_LAUNCH_CHECK();
}

X0NE_API int x0ne_moe_group(const int32_t* chosen, int pairs, int experts, int32_t* offsets, int32_t* listed, int32_t* tiles,
                            int max_tiles, int tile_m, int32_t* n_tiles_out, cudaStream_t stream) {
    X0NE_REQUIRE(pairs >= 0 && experts > 0 && tile_m > 0 && max_tiles >= x0ne_moe_max_tiles(pairs, experts, tile_m),
                 "moe_group: pairs %d experts %d tiles %d of %d", pairs, experts, max_tiles, tile_m);
    if (pairs == 0) return 0;
    const size_t smem = (size_t)(3 * experts + 2) * sizeof(int);
    X0NE_REQUIRE(smem <= 48 * 1024, "moe_group: %d experts are more than the kernel holds", experts);
    x0ne_launch(moe_group_kernel, dim3(1), dim3(1024), smem, stream, chosen, pairs, experts, offsets, listed, tiles, max_tiles, tile_m,
                n_tiles_out);
    X0NE_LAUNCH_CHECK();
}

// which = 0: up product with the squared ReLU (a: the rows [*, K], out: activation type [pairs][N]);
// which = 1: down product (a: the activations [pairs][K], out: float32 [pairs][N]).  w: [experts][N][K].
// which = 2: gated up product, silu(gate) * up (w: [experts][2 N][K], an expert's gate rows before its up rows, or, with
// pair_block > 0 (which divides N), in blocks of pair_block gate rows followed by the up rows of the same outputs).
X0NE_API int x0ne_moe_product(int which, const void* a, int64_t lda, const void* w, int dt, int N, int K, const int32_t* listed,
                              const int32_t* tiles, int max_tiles, int top, void* out, int pair_block, cudaStream_t stream) {
    X0NE_REQUIRE((which == 0 || which == 1 || which == 2) && N > 0 && K > 0 && lda >= K && top > 0 && max_tiles >= 0, "moe_product: N %d K %d lda %lld", N, K, (long long)lda);
    X0NE_REQUIRE(dt == X0NE_F32 || dt == X0NE_BF16, "moe_product: unknown dtype tag %d", dt);
    if (max_tiles == 0) return 0;
    X0NE_REQUIRE(max_tiles <= 65535, "moe_product: %d tiles in one launch", max_tiles);
    const dim3 grid((N + 63) / 64, max_tiles), block(256);
    if (dt == X0NE_F32) {
        if (which == 0) x0ne_launch(moe_product_kernel<float, 1>, grid, block, 0, stream, (const float*)a, lda, (const float*)w, N, K, listed, tiles, top, out, pair_block);
        else if (which == 2) x0ne_launch(moe_product_kernel<float, 2>, grid, block, 0, stream, (const float*)a, lda, (const float*)w, N, K, listed, tiles, top, out, pair_block);
        else x0ne_launch(moe_product_kernel<float, 0>, grid, block, 0, stream, (const float*)a, lda, (const float*)w, N, K, listed, tiles, top, out, pair_block);
    } else {
        if (which == 0) x0ne_launch(moe_product_kernel<bf16, 1>, grid, block, 0, stream, (const bf16*)a, lda, (const bf16*)w, N, K, listed, tiles, top, out, pair_block);
        else if (which == 2) x0ne_launch(moe_product_kernel<bf16, 2>, grid, block, 0, stream, (const bf16*)a, lda, (const bf16*)w, N, K, listed, tiles, top, out, pair_block);
        else x0ne_launch(moe_product_kernel<bf16, 0>, grid, block, 0, stream, (const bf16*)a, lda, (const bf16*)w, N, K, listed, tiles, top, out, pair_block);
    }
    X0NE_LAUNCH_CHECK();
}

X0NE_API int x0ne_moe_combine(const float* y, const void* x, int dt, const int32_t* chosen, const float* weights, int top, int experts,
                              const void* shared, const float* sgate, void* out, int n_rows, int hidden, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && hidden > 0 && top > 0 && experts >= 0, "moe_combine: rows %d hidden %d top %d", n_rows, hidden, top);
    if (n_rows == 0) return 0;
    if (hidden % 4 == 0 && top <= CMB_MAX_TOP && n_rows <= 65535 && (dt == X0NE_F32 || dt == X0NE_BF16) &&
        ((((uintptr_t)y | (uintptr_t)x | (uintptr_t)shared | (uintptr_t)out) & 15) == 0)) {
        const int threads = hidden / 4 >= 256 ? 256 : (hidden / 4 + 31) / 32 * 32;
        const dim3 grid((hidden / 4 + threads - 1) / threads, n_rows);
        if (dt == X0NE_F32)
            x0ne_launch(moe_combine_vec_kernel<float>, grid, dim3(threads), 0, stream, y, (const float*)x, chosen, weights, top, experts, (const float*)shared, sgate, (float*)out, hidden);
        else
            x0ne_launch(moe_combine_vec_kernel<bf16>, grid, dim3(threads), 0, stream, y, (const bf16*)x, chosen, weights, top, experts, (const bf16*)shared, sgate, (bf16*)out, hidden);
        X0NE_LAUNCH_CHECK();
    }
    if (dt == X0NE_F32)
        x0ne_launch(moe_combine_kernel<float>, dim3(n_rows), dim3(256), 0, stream, y, (const float*)x, chosen, weights, top, experts, (const float*)shared, sgate, (float*)out, hidden);
    else if (dt == X0NE_BF16)
        x0ne_launch(moe_combine_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, y, (const bf16*)x, chosen, weights, top, experts, (const bf16*)shared, sgate, (bf16*)out, hidden);
    else
        X0NE_REQUIRE(false, "moe_combine: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}
