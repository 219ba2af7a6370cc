// The experts' products of a routed feed-forward on the 5th-generation tensor cores, for passes with
// many (row, choice) pairs: the pairs of one expert lie together (moe.cu lists them), so a 128-row tile
// of one expert's pairs times a 256-row tile of that expert's weight is one tcgen05 accumulator, and
// the whole layer is one launch over a table of tiles that the grouping kernel wrote on the device.
//
//   up:   A = the rows gathered into the listed order [places][K] (moe_gather_rows), W = up weights
//         [experts x N][K]; the epilogue writes relu(.)^2 as bfloat16 to act[place][N]
//   down: A = act [places][K], W = down weights [experts x N][K]; the epilogue writes float32 to
//         y[pair][N], the pair looked up from the list (a row of the tile is one thread's)
//   gated up: W = [experts x N][K] with N = 2 x the experts' inner width, an expert's rows in blocks of 256: 128 gate
//         rows, then the 128 up rows of the same outputs; a tile's accumulator then holds a gate value and its up value
//         128 columns apart, and the epilogue writes silu(gate) * up as bfloat16 to act[place][N / 2]
//
// The pipeline is the one of gemm_tcgen05.cu: a copy thread (TMA, 128-byte swizzle, 4 stages), an MMA
// thread (accumulator double-buffered in tensor memory) and four epilogue warps; blocks are
// persistent over the tiles.  How many tiles are real is read from device memory (the launch is sized
// for the worst case), so the launch depends on the host only through sizes.  A tile's A rows past the
// expert's last pair and W rows past the expert's last output row are read (the next expert's, or
// zeros past the end) and their results dropped.  Every barrier wait is bounded; a wait that runs out
// sets its bit in `status`, and the kernel frees its tensor memory and returns.
#include "tcgen05.cuh"

#define MT_BM 128
#define MT_BN 256
#define MT_BK 64
#define MT_STAGES 4
#define MT_THREADS 192
#define MT_TMEM_COLS 512

struct MtShared {
    uint64_t full[MT_STAGES];
    uint64_t empty[MT_STAGES];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint32_t tmem_base;
    int failed;
};

#define MT_UP 0
#define MT_DOWN 1
#define MT_GATED 2

template <int MODE>
__global__ void __launch_bounds__(MT_THREADS) moe_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                            const __grid_constant__ CUtensorMap map_w, void* __restrict__ out,
                                                            int N, int K, const int32_t* __restrict__ listed,
                                                            const int32_t* __restrict__ tiles, const int32_t* __restrict__ n_real_p,
                                                            int max_tiles, int n_tiles_n, int* status) {
    extern __shared__ unsigned char mt_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(mt_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = MT_BM * 128, B_BYTES = MT_BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
    MtShared* sh = reinterpret_cast<MtShared*>(base + MT_STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + MT_BK - 1) / MT_BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < MT_STAGES; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh->accum_full[b], 1);
            mbar_init(&sh->accum_empty[b], 128);
        }
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&sh->tmem_base)),
                     "r"(MT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    pdl_wait();          // the table of tiles, the list and the A rows were written by the kernels before this one
    // the A rows were written with ordinary stores and are read by TMA: order the two proxies on this side as well
    asm volatile("fence.proxy.async;" ::: "memory");
    int n_real = n_real_p[0];
    if (n_real > max_tiles) n_real = max_tiles;
    const int total = n_real * n_tiles_n;      // tile id -> (m tile = id % n_real, n tile = id / n_real)

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < total && !sh->failed; tile += gridDim.x) {
                const int mt = tile % n_real, n0 = (tile / n_real) * MT_BN;
                const int e = tiles[3 * mt], first = tiles[3 * mt + 1];
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % MT_STAGES;
                    if (it >= MT_STAGES && !mbar_wait(&sh->empty[s], ((it / MT_STAGES) - 1) & 1, status, 1)) {
                        sh->failed = 1;
                        break;
                    }
                    unsigned char* a = base + s * STAGE_BYTES;
                    mbar_expect_tx(&sh->full[s], STAGE_BYTES);
                    tma_load_2d(a, &map_a, kb * MT_BK, first, &sh->full[s]);
                    tma_load_2d(a + A_BYTES, &map_w, kb * MT_BK, e * N + n0, &sh->full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N = 256, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
            int it = 0, t = 0;
            for (int tile = blockIdx.x; tile < total && !sh->failed; tile += gridDim.x, ++t) {
                const int ab = t & 1;
                const uint32_t acc_tmem = tmem + ab * 256;
                if (t >= 2 && !mbar_wait(&sh->accum_empty[ab], ((t >> 1) - 1) & 1, status, 4)) {
                    sh->failed = 1;
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % MT_STAGES;
                    if (!mbar_wait(&sh->full[s], (it / MT_STAGES) & 1, status, 2)) {
                        sh->failed = 1;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a = tc_smem(base + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                    for (int k = 0; k < MT_BK / 16; ++k)
                        tc_mma(acc_tmem, tc_desc(a + k * 32), tc_desc(b + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(&sh->empty[s]);
                }
                tc_commit(&sh->accum_full[ab]);
            }
        }
    } else {
        const int quarter = warp & 3;
        int t = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++t) {
            const int ab = t & 1;
            const int mt = tile % n_real, n0 = (tile / n_real) * MT_BN;
            const int first = tiles[3 * mt + 1], count = tiles[3 * mt + 2];
            const int r = quarter * 32 + lane;
            int64_t row = -1;                              // the output row of this thread, or none
            if (r < count) row = MODE != MT_DOWN ? (int64_t)(first + r) : (int64_t)listed[first + r];
            if (!mbar_wait(&sh->accum_full[ab], (t >> 1) & 1, status, 3) || sh->failed) {
                sh->failed = 1;
                break;
            }
            tc_fence_after();
            const uint32_t trow = tmem + ab * 256 + ((uint32_t)(quarter * 32) << 16);
            if (MODE == MT_GATED) {
                // columns c and 128 + c of the tile are the gate and the up value of output n0 / 2 + c (N is a multiple of 256)
                const int half = N / 2;
#pragma unroll 1
                for (int c = 0; c < MT_BN / 64; ++c) {
                    float v[32], u[32];
                    tc_ld32(trow + c * 32, v);
                    tc_ld32(trow + MT_BN / 2 + c * 32, u);
                    if (row < 0) continue;
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.0f + __expf(-v[i])) * u[i];
                    bf16* dst = (bf16*)out + row * half + n0 / 2 + c * 32;
                    if ((((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) tc_store8(dst + i, v + i);
                    } else {
                        for (int i = 0; i < 32; ++i) dst[i] = __float2bfloat16_rn(v[i]);
                    }
                }
                tc_fence_before();
                mbar_arrive(&sh->accum_empty[ab]);
                continue;
            }
#pragma unroll 1
            for (int c = 0; c < MT_BN / 32; ++c) {
                const int n = n0 + c * 32;
                if (n >= N) break;                          // (uniform over the warp)
                float v[32];
                tc_ld32(trow + c * 32, v);
                if (row < 0) continue;
                if (MODE == MT_UP) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float x = fmaxf(v[i], 0.f);
                        v[i] = x * x;
                    }
                    bf16* dst = (bf16*)out + row * N + n;
                    if (n + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) tc_store8(dst + i, v + i);
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (n + i < N) dst[i] = __float2bfloat16_rn(v[i]);
                    }
                } else {
                    float* dst = (float*)out + row * N + n;
                    if (n + 32 <= N && (((uintptr_t)dst) & 31) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) tc_store8(dst + i, v + i);
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (n + i < N) dst[i] = v[i];
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&sh->accum_empty[ab]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(MT_TMEM_COLS) : "memory");
    }
}

// xs[place] = x[listed[place] / top] for the places that hold a pair (their number is offsets[experts]).
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, int K, const int32_t* __restrict__ listed,
                                       const int32_t* __restrict__ offsets, int experts, int top, bf16* __restrict__ xs) {
    pdl_prologue();
    const int place = blockIdx.x;
    if (place >= offsets[experts]) return;
    const bf16* src = x + (int64_t)(listed[place] / top) * K;
    bf16* dst = xs + (int64_t)place * K;
    if (K % 8 == 0 && ((((uintptr_t)x | (uintptr_t)xs) & 15) == 0)) {
        for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < K; i += blockDim.x) dst[i] = src[i];
    }
}

X0NE_API int x0ne_moe_tc_tile_rows() { return MT_BM; }

X0NE_API int x0ne_moe_gather_rows(const void* x, int K, const int32_t* listed, const int32_t* offsets, int experts, int top,
                                  void* xs, int pairs, cudaStream_t stream) {
    X0NE_REQUIRE(K > 0 && experts > 0 && top > 0 && pairs >= 0, "moe_gather: K %d experts %d top %d", K, experts, top);
    if (pairs == 0) return 0;
    x0ne_launch(moe_gather_rows_kernel, dim3(pairs), dim3(K >= 2048 ? 256 : 128), 0, stream, (const bf16*)x, K, listed, offsets, experts,
                top, (bf16*)xs);
    X0NE_LAUNCH_CHECK();
}

// which 0: up (a: gathered rows [a_rows][K], out: bfloat16 act [places][N]); which 1: down (a: act [a_rows][K], out:
// float32 y [pairs][N]); which 2: gated up (a as for 0, w rows in blocks of 128 gate and 128 up rows, N a multiple of 256,
// out: bfloat16 act [places][N / 2]).  w: [experts][N][K] bfloat16.  tiles: [max_tiles][3] from the grouping kernel run with
// tiles of 128 pairs; n_real: how many of them are real (device memory).
X0NE_API int x0ne_moe_product_tc(int which, const void* a, int64_t a_rows, const void* w, int experts, int N, int K,
                                 const int32_t* listed, const int32_t* tiles, const int32_t* n_real, int max_tiles, void* out,
                                 int* status, cudaStream_t stream) {
    X0NE_REQUIRE((which == 0 || which == 1 || which == 2) && experts > 0 && N > 0 && K > 0 && K % 8 == 0 && a_rows > 0 && max_tiles >= 0,
                 "moe_product_tc: experts %d N %d K %d (K must be a multiple of 8)", experts, N, K);
    X0NE_REQUIRE(which != 2 || N % MT_BN == 0, "moe_product_tc: gated experts of %d rows (blocks of %d)", N, MT_BN);
    X0NE_REQUIRE(status != nullptr && n_real != nullptr, "moe_product_tc: no status word or no tile count");
    X0NE_REQUIRE((((uintptr_t)a | (uintptr_t)w) & 15) == 0, "moe_product_tc: operands are not 16-byte aligned");
    if (max_tiles == 0) return 0;
    CUtensorMap map_a, map_w;
    if (int e = x0ne_tc_make_map(&map_a, a, a_rows, K, MT_BM)) return e;
    if (int e = x0ne_tc_make_map(&map_w, w, (int64_t)experts * N, K, MT_BN)) return e;
    const size_t smem = (size_t)MT_STAGES * (MT_BM * 128 + MT_BN * 128) + sizeof(MtShared) + 1024;
    static OncePerDevice configured;
    if (configured.need()) {
        cudaError_t e1 = cudaFuncSetAttribute(moe_tc_kernel<MT_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaError_t e2 = cudaFuncSetAttribute(moe_tc_kernel<MT_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaError_t e3 = cudaFuncSetAttribute(moe_tc_kernel<MT_GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) {
            x0ne_set_error("moe_product_tc: cannot set %zu bytes of shared memory", smem);
            return (int)(e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3));
        }
        configured.done();
    }
    const int n_tiles_n = (N + MT_BN - 1) / MT_BN;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 1;
    const int64_t worst = (int64_t)max_tiles * n_tiles_n;
    const int grid = worst < sms ? (int)worst : sms;
    // Launched without the early-start attribute: the kernel before it writes, with ordinary stores at its very end, the rows
    // this one reads by TMA a moment later.  Replayed from a graph with the early start, short prompt passes with many padding
    // rows gave other logits than the same launches made one by one (which leave more time between the two kernels); with a
    // plain launch and the proxy fence in the kernel they give the same bits.  The kernel still lets its own successor start early.
    if (which == 0)
        moe_tc_kernel<MT_UP><<<grid, MT_THREADS, smem, stream>>>(map_a, map_w, out, N, K, listed, tiles, n_real, max_tiles, n_tiles_n, status);
    else if (which == 2)
        moe_tc_kernel<MT_GATED><<<grid, MT_THREADS, smem, stream>>>(map_a, map_w, out, N, K, listed, tiles, n_real, max_tiles, n_tiles_n, status);
    else
        moe_tc_kernel<MT_DOWN><<<grid, MT_THREADS, smem, stream>>>(map_a, map_w, out, N, K, listed, tiles, n_real, max_tiles, n_tiles_n, status);
    X0NE_LAUNCH_CHECK();
}
