// Attention over the paged cache in bfloat16 for the shapes and rules the fixed-shape kernels do
// not take: keys and values of different widths (any width: rows are padded with zeros to a
// multiple of 16 in shared memory), values that are the leading part of the key rows (a latent
// cache read by every head), a chunked mask, a sliding window, first keys that stay visible whatever
// the window, a per-head sink in the softmax denominator, a per-head slope times the distance i - j taken off the
// scaled score, a sigmoid gate on the output per (row, head) or per (row, head, value), and results written as float32.
//
// Both kernels are flash attention on `mma.sync` m16n8k16 with float32 accumulation.  Scores,
// maxima, sums and weights are float32; for the product with the values a weight p is split into
// bfloat16(p) and bfloat16(p - bfloat16(p)), two products into the same float32 accumulator, so
// the weights enter with 16 bits of mantissa instead of 8 (what is left is below the rounding of
// the bfloat16 values themselves).
//
//   prefill: a block takes a tile of up to 128 consecutive rows of one sequence and one q head;
//            8 warps x 16 rows; key pages of 64 positions are staged in shared memory.
//   decode:  a block takes one row (sequence), one kv head, up to 16 q heads of its group (the MMA
//            rows) and one split of the row's pages; 4 warps take 16 keys of every page each and
//            merge at the end; several splits leave partial results in scratch that a second
//            kernel merges in split order (same bits on every call).
#include "common.cuh"

#define FX_PAGE 64
#define FX_TILE_ROWS 128
#define FX_LOG2E 1.4426950408889634f
#ifndef FX_DECODE_STAGES
#define FX_DECODE_STAGES 2      // stages of (key tile, value tile) a decode block copies ahead through
#endif

__device__ __forceinline__ void fx_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fx_ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void fx_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
// 16 bytes from global to shared memory without passing through registers; zeros when `valid` is false
// (nothing is read then: `src` only has to be an address of global memory)
__device__ __forceinline__ void fx_cp16(bf16* dst, const bf16* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void fx_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fx_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A result at place i (counted in values) of the output: bfloat16, or float32 for a caller that asked for it.
__device__ __forceinline__ void fx_store(bf16* out, int64_t i, float v, bool f32) {
    if (f32) reinterpret_cast<float*>(out)[i] = v;
    else out[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ uint32_t fx_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// bfloat16(p) and the bfloat16 of what that rounding lost, for two weights at once
__device__ __forceinline__ void fx_split(float p0, float p1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);          // p0 in the low half
    hi = *reinterpret_cast<const uint32_t*>(&hv);
    lo = fx_pack(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
}

// Copies rows [0, n_rows) of `d` values (row r at src + r * src_ld) into dst rows of `stride` values,
// zero where r is outside [r_lo, r_hi] or src is null, and zero in the columns d .. dp-1.
__device__ __forceinline__ void fx_load_rows(bf16* dst, int stride, const bf16* src, int64_t src_ld, int n_rows, int r_lo, int r_hi,
                                             int d, int dp, int tid, int nthreads) {
    const bool vec = (d % 8 == 0) && (src_ld % 8 == 0) && ((((uintptr_t)src) & 15) == 0);
    if (vec) {
        const int per_row = dp / 8;
        for (int i = tid; i < n_rows * per_row; i += nthreads) {
            const int r = i / per_row, c = (i % per_row) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (src != nullptr && r >= r_lo && r <= r_hi && c < d) v = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
            *reinterpret_cast<uint4*>(dst + r * stride + c) = v;
        }
    } else {
        for (int i = tid; i < n_rows * dp; i += nthreads) {
            const int r = i / dp, c = i % dp;
            bf16 v = __float2bfloat16_rn(0.f);
            if (src != nullptr && r >= r_lo && r <= r_hi && c < d) v = src[r * src_ld + c];
            dst[r * stride + c] = v;
        }
    }
}

// Where a thread starts and how it steps when a block shares the 16-byte pieces of a tile's rows: worked
// out once per kernel (the divisions), used for every page.
struct FxPieces {
    int r0, c0, dr, dc, per_row;
};
__device__ __forceinline__ FxPieces fx_pieces(int dp, int tid, int nthreads) {
    FxPieces p;
    p.per_row = dp / 8;
    p.r0 = tid / p.per_row;
    p.c0 = tid % p.per_row;
    p.dr = nthreads / p.per_row;
    p.dc = nthreads % p.per_row;
    return p;
}

// The same through cp.async where rows can be copied 16 bytes at a time (the caller commits and waits);
// other shapes, and a missing source, are written with plain stores.  `safe` is any address of global memory.
__device__ __forceinline__ void fx_load_rows_async(bf16* dst, int stride, const bf16* src, int64_t src_ld, int n_rows, int r_lo, int r_hi,
                                                   int d, int dp, int tid, int nthreads, const bf16* safe, const FxPieces& pc) {
    const bool vec = src != nullptr && (d % 8 == 0) && (src_ld % 8 == 0) && ((((uintptr_t)src) & 15) == 0);
    if (!vec) {
        fx_load_rows(dst, stride, src, src_ld, n_rows, r_lo, r_hi, d, dp, tid, nthreads);
        return;
    }
    int r = pc.r0, c8 = pc.c0;
    while (r < n_rows) {
        const int c = c8 * 8;
        const bool ok = r >= r_lo && r <= r_hi && c < d;
        fx_cp16(dst + r * stride + c, ok ? src + r * src_ld + c : safe, ok);
        r += pc.dr;
        c8 += pc.dc;
        if (c8 >= pc.per_row) {
            c8 -= pc.per_row;
            ++r;
        }
    }
}

// The physical page of a sequence's logical page, or -1.
__device__ __forceinline__ int fx_page(const PagedCache& c, int slot, int logical) {
    if (slot < 0) return -1;
    const int page = c.page_table[(int64_t)slot * c.table_stride + logical % c.ring_pages];
    return (page < 0 || page >= c.n_pages) ? -1 : page;
}

__device__ __forceinline__ int fx_first_key(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, pos - pos % chunk);
    return lo;
}

struct FxShape {
    int dk, dkp, vd, vdp;     // key and value widths, and the same padded to multiples of 16
    int ks, vs;               // shared-memory row strides (values) of the key and value tiles
};

// S (16 rows of this warp x 8 n-tiles of 8 keys, starting at key tile row `key0`) = Q K^T.
template <int NT>
__device__ __forceinline__ void fx_scores(float (*s)[4], const bf16* qs, const bf16* ks, int stride, int dkp, int key0, int lane) {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    // ldmatrix addresses of this lane: the query fragment (rows 0-7 / 8-15, k 0-7 / 8-15) and the key
    // fragments of two n-tiles at once (keys 8n.. / 8(n+1).., k 0-7 / 8-15)
    const bf16* qa = qs + ((mi & 1) * 8 + r) * stride + (mi >> 1) * 8;
    const bf16* ka = ks + (key0 + (mi >> 1) * 8 + r) * stride + (mi & 1) * 8;
    for (int kk = 0; kk < dkp; kk += 16) {
        uint32_t a0, a1, a2, a3;
        fx_ldmatrix_x4(a0, a1, a2, a3, qa + kk);
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            uint32_t b0, b1, b2, b3;
            fx_ldmatrix_x4(b0, b1, b2, b3, ka + 8 * n * stride + kk);
            fx_mma(s[n], a0, a1, a2, a3, b0, b1);
            fx_mma(s[n + 1], a0, a1, a2, a3, b2, b3);
        }
    }
}

// O (16 rows x DVT n-tiles of 8 values) += P V for KB blocks of 16 keys starting at value tile row `key0`;
// `p` holds the weights of those keys as score fragments (2 n-tiles per block of 16 keys).
template <int DVT, int KB>
__device__ __forceinline__ void fx_accumulate(float (*o)[4], const float (*p)[4], const bf16* vs, int stride, int key0, int lane) {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
        uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
        fx_split(p[2 * kb][0], p[2 * kb][1], h0, l0);
        fx_split(p[2 * kb][2], p[2 * kb][3], h1, l1);
        fx_split(p[2 * kb + 1][0], p[2 * kb + 1][1], h2, l2);
        fx_split(p[2 * kb + 1][2], p[2 * kb + 1][3], h3, l3);
        const bf16* row = vs + (key0 + 16 * kb + (mi & 1) * 8 + r) * stride + (mi >> 1) * 8;
#pragma unroll
        for (int n = 0; n < DVT; n += 2) {
            uint32_t b0, b1, b2, b3;
            fx_ldmatrix_x4_trans(b0, b1, b2, b3, row + 8 * n);
            fx_mma(o[n], h0, h1, h2, h3, b0, b1);
            fx_mma(o[n], l0, l1, l2, l3, b0, b1);
            fx_mma(o[n + 1], h0, h1, h2, h3, b2, b3);
            fx_mma(o[n + 1], l0, l1, l2, l3, b2, b3);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// prefill
// ------------------------------------------------------------------------------------------------
template <int DVT>
__global__ void __launch_bounds__(256, DVT > 16 ? 1 : 2)
flex_prefill_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, PagedCache cache, const int32_t* __restrict__ tile_seq,
                    const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ seq_first_row,
                    const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_pos0, int q_heads, float scale,
                    int window, AttnExtra ex, FxShape sh) {
    extern __shared__ __align__(16) unsigned char fx_smem[];
    // queries, then two stages of (key tile, value tile): the next page is copied while this one is used
    bf16* qs = reinterpret_cast<bf16*>(fx_smem);
    bf16* ks0 = qs + FX_TILE_ROWS * sh.ks;
    const int stage_elems = FX_PAGE * sh.ks + (ex.v_from_k > 0 ? 0 : FX_PAGE * sh.vs);
    const int vstride = ex.v_from_k > 0 ? sh.ks : sh.vs;
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, head = blockIdx.y;
    const int kh = head / (q_heads / cache.kv_heads);
    const int seq = tile_seq[tile], row0 = tile_row0[tile];
    const int slot = seq_slot[seq];
    const int pos0 = seq_pos0[seq] + (row0 - seq_first_row[seq]);
    const int n_rows = min(FX_TILE_ROWS, seq_first_row[seq + 1] - row0);
    const float sink2 = ex.sink != nullptr ? ex.sink[head] * FX_LOG2E : -INFINITY;
    const bool sloped = ex.slope != nullptr;
    const float sl2 = sloped ? ex.slope[head] * FX_LOG2E : 0.f;       // taken off per position of distance, in the exp2 domain
    pdl_wait();
    const int64_t q_ld = ex.q_ld > 0 ? ex.q_ld : (int64_t)q_heads * sh.dk;
    const bf16* safe = (const bf16*)cache.base;
    const FxPieces pk = fx_pieces(sh.dkp, tid, 256), pv = fx_pieces(sh.vdp, tid, 256);
    fx_load_rows_async(qs, sh.ks, q + (int64_t)row0 * q_ld + (int64_t)head * sh.dk, q_ld, FX_TILE_ROWS, 0, n_rows - 1, sh.dk, sh.dkp, tid, 256, safe, pk);

    const float sc2 = scale * FX_LOG2E;
    const int r_a = warp * 16 + g, r_b = r_a + 8;                  // this thread's two rows of the tile
    const int pos_a = pos0 + r_a, pos_b = pos0 + r_b;
    const int lo_a = fx_first_key(pos_a, window, ex.chunk), lo_b = fx_first_key(pos_b, window, ex.chunk);
    const bool ok_a = r_a < n_rows, ok_b = r_b < n_rows;
    const int warp_last = pos0 + min(warp * 16 + 15, n_rows - 1);  // the largest position a row of this warp has
    const int warp_first_key = fx_first_key(pos0 + warp * 16, window, ex.chunk);   // first keys only grow along the rows
    const bool warp_all_rows = warp * 16 + 15 < n_rows;
    const int warp_first_pos = pos0 + warp * 16;                                    // the smallest position of this warp's rows
    const int warp_last_key = fx_first_key(pos0 + warp * 16 + 15, window, ex.chunk);   // the largest first key of them
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[DVT][4];
#pragma unroll
    for (int n = 0; n < DVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    const int key_lo = fx_first_key(pos0, window, ex.chunk), key_hi = pos0 + n_rows - 1;
    const int64_t k_head = (int64_t)kh * cache.page_size * sh.dk;
    const int64_t v_head = (int64_t)cache.kv_heads * cache.page_size * sh.dk + (int64_t)kh * cache.page_size * sh.vd;
    const int pg_first = key_lo / FX_PAGE, pg_last = key_hi / FX_PAGE;
    // pages of kept first keys that lie wholly before the first page of the window come first in the walk
    const int n_kept = min((ex.keep_first + FX_PAGE - 1) / FX_PAGE, pg_first);
    const int n_walk = n_kept + pg_last - pg_first + 1;
    auto issue = [&](int pg, int stage) -> bool {       // copies page pg into a stage; false if the sequence has no such page
        const int page = fx_page(cache, slot, pg);
        const bf16* pb = page >= 0 ? (const bf16*)cache.base + (int64_t)page * cache.page_stride : nullptr;
        bf16* kd = ks0 + stage * stage_elems;
        fx_load_rows_async(kd, sh.ks, pb ? pb + k_head : nullptr, sh.dk, FX_PAGE, 0, key_hi - pg * FX_PAGE, sh.dk, sh.dkp, tid, 256, safe, pk);
        if (ex.v_from_k <= 0)
            fx_load_rows_async(kd + FX_PAGE * sh.ks, sh.vs, pb ? pb + v_head : nullptr, sh.vd, FX_PAGE, 0, key_hi - pg * FX_PAGE, sh.vd, sh.vdp, tid, 256, safe, pv);
        fx_cp_commit();
        return pb != nullptr;
    };
    bool have = issue(n_kept > 0 ? 0 : pg_first, 0);
    for (int it = 0; it < n_walk; ++it) {
        const int pg = it < n_kept ? it : pg_first + it - n_kept;
        const int j0 = pg * FX_PAGE;
        const int stage = it & 1;
        const bf16* ks = ks0 + stage * stage_elems;
        const bf16* vs = ex.v_from_k > 0 ? ks : ks + FX_PAGE * sh.ks;
        const bool here = have;
        if (it + 1 < n_walk) {
            have = issue(it + 1 < n_kept ? it + 1 : pg_first + it + 1 - n_kept, stage ^ 1);       // (the stage was last read two pages ago; the barrier at the end of that page covers it)
            fx_cp_wait<1>();
        } else {
            fx_cp_wait<0>();
        }
        __syncthreads();          // this page's tile (and, the first time, the queries) is complete for every warp
        const bool skip = !here;
        if (warp * 16 >= n_rows || j0 > warp_last || (j0 + FX_PAGE <= warp_first_key && j0 >= ex.keep_first) || skip) {   // nothing of this page for this warp
            __syncthreads();
            continue;
        }
        float s[8][4];
        fx_scores<8>(s, qs + warp * 16 * sh.ks, ks, sh.ks, sh.dkp, 0, lane);
        float mx_a = -INFINITY, mx_b = -INFINITY;
        if (warp_all_rows && j0 + FX_PAGE - 1 <= warp_first_pos && (j0 >= warp_last_key || j0 + FX_PAGE <= ex.keep_first)) {
            // every key of the page is seen by every row of this warp: no comparisons
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] *= sc2;
                if (sloped) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = j0 + 8 * n + 2 * t + e;
                        s[n][e] -= sl2 * (float)(pos_a - j);
                        s[n][2 + e] -= sl2 * (float)(pos_b - j);
                    }
                }
                mx_a = fmaxf(mx_a, fmaxf(s[n][0], s[n][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[n][2], s[n][3]));
            }
        } else {
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + 8 * n + 2 * t + e;
                    float sa = s[n][e] * sc2, sb = s[n][2 + e] * sc2;
                    if (sloped) {
                        sa -= sl2 * (float)(pos_a - j);
                        sb -= sl2 * (float)(pos_b - j);
                    }
                    s[n][e] = (ok_a && j <= pos_a && (j >= lo_a || j < ex.keep_first)) ? sa : -INFINITY;
                    s[n][2 + e] = (ok_b && j <= pos_b && (j >= lo_b || j < ex.keep_first)) ? sb : -INFINITY;
                    mx_a = fmaxf(mx_a, s[n][e]);
                    mx_b = fmaxf(mx_b, s[n][2 + e]);
                }
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float al_a = exp2f(m_a - ref_a), al_b = exp2f(m_b - ref_b);
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            s[n][0] = exp2f(s[n][0] - ref_a); s[n][1] = exp2f(s[n][1] - ref_a);
            s[n][2] = exp2f(s[n][2] - ref_b); s[n][3] = exp2f(s[n][3] - ref_b);
            sum_a += s[n][0] + s[n][1];
            sum_b += s[n][2] + s[n][3];
        }
        l_a = l_a * al_a + sum_a;
        l_b = l_b * al_b + sum_b;
        m_a = mn_a;
        m_b = mn_b;
        if (!__all_sync(0xffffffffu, al_a == 1.f && al_b == 1.f)) {      // (once the maxima have settled nothing is rescaled)
#pragma unroll
            for (int n = 0; n < DVT; ++n) { o[n][0] *= al_a; o[n][1] *= al_a; o[n][2] *= al_b; o[n][3] *= al_b; }
        }
        fx_accumulate<DVT, 4>(o, s, vs, vstride, 0, lane);
        __syncthreads();          // every warp is done with this stage before the page after next is copied into it
    }
    // the row's sum over its four threads, the sink, the gate, and out
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    float f_a = 1.f, f_b = 1.f;
    if (ex.sink != nullptr) {
        const float mf_a = fmaxf(m_a, sink2), mf_b = fmaxf(m_b, sink2);
        f_a = exp2f(m_a - mf_a); f_b = exp2f(m_b - mf_b);
        l_a = l_a * f_a + exp2f(sink2 - mf_a);
        l_b = l_b * f_b + exp2f(sink2 - mf_b);
    }
    f_a *= l_a > 0.f ? 1.0f / l_a : 0.f;
    f_b *= l_b > 0.f ? 1.0f / l_b : 0.f;
    const bool wide = ex.gate != nullptr && ex.gate_wide > 0;       // a gate per value of the head, not one per head
    if (ex.gate != nullptr && !wide) {
        const bf16* gt = (const bf16*)ex.gate;
        if (ok_a) f_a *= 1.0f / (1.0f + expf(-__bfloat162float(gt[(int64_t)(row0 + r_a) * ex.gate_ld + head])));
        if (ok_b) f_b *= 1.0f / (1.0f + expf(-__bfloat162float(gt[(int64_t)(row0 + r_b) * ex.gate_ld + head])));
    }
    const bf16* ga = (const bf16*)ex.gate + (int64_t)(row0 + r_a) * ex.gate_ld + (int64_t)head * sh.vd;
    const bf16* gb = (const bf16*)ex.gate + (int64_t)(row0 + r_b) * ex.gate_ld + (int64_t)head * sh.vd;
    const int64_t oa = ((int64_t)(row0 + r_a) * q_heads + head) * sh.vd, ob = ((int64_t)(row0 + r_b) * q_heads + head) * sh.vd;
    const bool f32 = ex.out_f32 > 0;
#pragma unroll
    for (int n = 0; n < DVT; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int c = 8 * n + 2 * t + e;
            if (c < sh.vd) {
                if (wide) {
                    if (ok_a) fx_store(out, oa + c, o[n][e] * f_a * (1.0f / (1.0f + expf(-__bfloat162float(ga[c])))), f32);
                    if (ok_b) fx_store(out, ob + c, o[n][2 + e] * f_b * (1.0f / (1.0f + expf(-__bfloat162float(gb[c])))), f32);
                } else {
                    if (ok_a) fx_store(out, oa + c, o[n][e] * f_a, f32);
                    if (ok_b) fx_store(out, ob + c, o[n][2 + e] * f_b, f32);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// decode
// ------------------------------------------------------------------------------------------------
// Partial result of a (row, kv head, head chunk) unit for one split: per item (q head) the maximum
// (in the exp2 domain), the sum and vdp accumulated values: 16 x (vdp + 2) floats.
template <int DVT>
__global__ void __launch_bounds__(128)
flex_decode_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, PagedCache cache, const int32_t* __restrict__ row_slot,
                   const int32_t* __restrict__ row_pos, int q_heads, float scale, int window, AttnExtra ex, FxShape sh,
                   int chunks, int splits, float* __restrict__ scratch) {
    extern __shared__ __align__(16) unsigned char fx_smem[];
    bf16* qs = reinterpret_cast<bf16*>(fx_smem);
    bf16* ks0 = qs + 16 * sh.ks;
    const int stage_elems = FX_PAGE * sh.ks + (ex.v_from_k > 0 ? 0 : FX_PAGE * sh.vs);
    const int vstride = ex.v_from_k > 0 ? sh.ks : sh.vs;
    float* mg = reinterpret_cast<float*>(ks0);         // the warps' partial results meet here at the end
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int group = q_heads / cache.kv_heads;
    const int unit = blockIdx.x, split = blockIdx.y;
    const int chunk_i = unit % chunks, kh = (unit / chunks) % cache.kv_heads, row = unit / (chunks * cache.kv_heads);
    const int slot = row_slot[row], pos = row_pos[row];
    const int head0 = kh * group + chunk_i * 16, n_items = min(16, group - chunk_i * 16);
    pdl_wait();
    const int64_t q_ld = ex.q_ld > 0 ? ex.q_ld : (int64_t)q_heads * sh.dk;
    const bf16* safe = (const bf16*)cache.base;
    const FxPieces pk = fx_pieces(sh.dkp, tid, 128), pv = fx_pieces(sh.vdp, tid, 128);
    fx_load_rows_async(qs, sh.ks, q + (int64_t)row * q_ld + (int64_t)head0 * sh.dk, sh.dk, 16, 0, n_items - 1, sh.dk, sh.dkp, tid, 128, safe, pk);

    const float sc2 = scale * FX_LOG2E;
    // the distance slopes of this thread's two items (q heads head0 + g and head0 + g + 8), in the exp2 domain
    const bool sloped = ex.slope != nullptr;
    const float sl_a = sloped && g < n_items ? ex.slope[head0 + g] * FX_LOG2E : 0.f;
    const float sl_b = sloped && g + 8 < n_items ? ex.slope[head0 + g + 8] * FX_LOG2E : 0.f;
    const int key_lo = fx_first_key(pos, window, ex.chunk);
    const int pg_lo = key_lo / FX_PAGE, pg_hi = slot >= 0 ? pos / FX_PAGE : pg_lo - 1;
    // the walk: pages of kept first keys that lie wholly before the window's first page, then the window's pages
    const int n_kept = slot >= 0 ? min((ex.keep_first + FX_PAGE - 1) / FX_PAGE, pg_lo) : 0;
    const int n_walk = n_kept + pg_hi - pg_lo + 1;
    const int per = (n_walk + splits - 1) / splits;
    const int it_a = split * per, it_b = min(n_walk - 1, it_a + per - 1);
    auto page_at = [&](int it) -> int { return it < n_kept ? it : pg_lo + it - n_kept; };
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[DVT][4];
#pragma unroll
    for (int n = 0; n < DVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const int64_t k_head = (int64_t)kh * cache.page_size * sh.dk;
    const int64_t v_head = (int64_t)cache.kv_heads * cache.page_size * sh.dk + (int64_t)kh * cache.page_size * sh.vd;
    auto issue = [&](int pg, int stage) -> bool {
        const int page = fx_page(cache, slot, pg);
        const bf16* pb = page >= 0 ? (const bf16*)cache.base + (int64_t)page * cache.page_stride : nullptr;
        bf16* kd = ks0 + stage * stage_elems;
        fx_load_rows_async(kd, sh.ks, pb ? pb + k_head : nullptr, sh.dk, FX_PAGE, 0, pos - pg * FX_PAGE, sh.dk, sh.dkp, tid, 128, safe, pk);
        if (ex.v_from_k <= 0)
            fx_load_rows_async(kd + FX_PAGE * sh.ks, sh.vs, pb ? pb + v_head : nullptr, sh.vd, FX_PAGE, 0, pos - pg * FX_PAGE, sh.vd, sh.vdp, tid, 128, safe, pv);
        fx_cp_commit();
        return pb != nullptr;
    };
    // FX_DECODE_STAGES - 1 pages are on their way while one is used; a group is committed for every page
    // slot, also an empty one, so that "all but the newest FX_DECODE_STAGES - 1 groups" is always this page's
    unsigned have = 0;                       // bit s: the page in stage s exists
    for (int i = 0; i < FX_DECODE_STAGES - 1; ++i) {
        if (it_a + i <= it_b) have |= issue(page_at(it_a + i), i) ? 1u << i : 0u;
        else fx_cp_commit();
    }
    for (int it = it_a; it <= it_b; ++it) {
        const int j0 = page_at(it) * FX_PAGE;
        const int stage = (it - it_a) % FX_DECODE_STAGES;
        const bf16* ks = ks0 + stage * stage_elems;
        const bf16* vs = ex.v_from_k > 0 ? ks : ks + FX_PAGE * sh.ks;
        const int ahead = it + FX_DECODE_STAGES - 1, ahead_stage = (ahead - it_a) % FX_DECODE_STAGES;
        have &= ~(1u << ahead_stage);        // (that stage was read one page ago; the barrier at that page's end covers it)
        if (ahead <= it_b) have |= issue(page_at(ahead), ahead_stage) ? 1u << ahead_stage : 0u;
        else fx_cp_commit();
        fx_cp_wait<FX_DECODE_STAGES - 1>();
        __syncthreads();
        const bool here = (have >> stage) & 1u;
        const int jw = j0 + 16 * warp;           // this warp's 16 keys of the page
        if (!here || jw > pos || (jw + 16 <= key_lo && jw >= ex.keep_first)) {
            __syncthreads();
            continue;
        }
        float s[2][4];
        fx_scores<2>(s, qs, ks, sh.ks, sh.dkp, 16 * warp, lane);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = jw + 8 * n + 2 * t + e;
                const bool vis = j <= pos && (j >= key_lo || j < ex.keep_first);
                float sa = s[n][e] * sc2, sb = s[n][2 + e] * sc2;
                if (sloped) {
                    sa -= sl_a * (float)(pos - j);
                    sb -= sl_b * (float)(pos - j);
                }
                s[n][e] = vis ? sa : -INFINITY;
                s[n][2 + e] = vis ? sb : -INFINITY;
            }
        }
        float mx_a = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx_b = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float al_a = exp2f(m_a - ref_a), al_b = exp2f(m_b - ref_b);
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            s[n][0] = exp2f(s[n][0] - ref_a); s[n][1] = exp2f(s[n][1] - ref_a);
            s[n][2] = exp2f(s[n][2] - ref_b); s[n][3] = exp2f(s[n][3] - ref_b);
            sum_a += s[n][0] + s[n][1];
            sum_b += s[n][2] + s[n][3];
        }
        l_a = l_a * al_a + sum_a;
        l_b = l_b * al_b + sum_b;
        m_a = mn_a;
        m_b = mn_b;
        if (!__all_sync(0xffffffffu, al_a == 1.f && al_b == 1.f)) {      // (once the maxima have settled nothing is rescaled)
#pragma unroll
            for (int n = 0; n < DVT; ++n) { o[n][0] *= al_a; o[n][1] *= al_a; o[n][2] *= al_b; o[n][3] *= al_b; }
        }
        fx_accumulate<DVT, 1>(o, s, vs, vstride, 16 * warp, lane);
        __syncthreads();
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    // the four warps' results -> shared memory [warp][item][vdp + 2]
    fx_cp_wait<0>();
    __syncthreads();
    const int ps = sh.vdp + 2;
    {
        float* wa = mg + ((int64_t)warp * 16 + g) * ps;
        float* wb = mg + ((int64_t)warp * 16 + g + 8) * ps;
        if (t == 0) { wa[0] = m_a; wa[1] = l_a; wb[0] = m_b; wb[1] = l_b; }
#pragma unroll
        for (int n = 0; n < DVT; ++n) {
            wa[2 + 8 * n + 2 * t] = o[n][0]; wa[2 + 8 * n + 2 * t + 1] = o[n][1];
            wb[2 + 8 * n + 2 * t] = o[n][2]; wb[2 + 8 * n + 2 * t + 1] = o[n][3];
        }
    }
    __syncthreads();
    // merge in warp order; thread = (item, a stripe of columns)
    const int item = tid >> 3, c0 = tid & 7;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mg[((int64_t)w * 16 + item) * ps]);
    const float ref = mm == -INFINITY ? 0.f : mm;
    float f[4], ll = 0.f;
    for (int w = 0; w < 4; ++w) {
        f[w] = exp2f(mg[((int64_t)w * 16 + item) * ps] - ref);
        ll += mg[((int64_t)w * 16 + item) * ps + 1] * f[w];
    }
    if (splits > 1) {
        float* dst = scratch + (((int64_t)unit * splits + split) * 16 + item) * ps;
        if (c0 == 0) { dst[0] = mm; dst[1] = ll; }
        for (int c = c0; c < sh.vdp; c += 8) {
            float acc = 0.f;
            for (int w = 0; w < 4; ++w) acc += mg[((int64_t)w * 16 + item) * ps + 2 + c] * f[w];
            dst[2 + c] = acc;
        }
        return;
    }
    if (item >= n_items) return;
    const int head = head0 + item;
    float fin = 1.f;
    if (ex.sink != nullptr) {
        const float sink2 = ex.sink[head] * FX_LOG2E;
        const float mf = fmaxf(mm, sink2);
        fin = exp2f(mm - mf);
        ll = ll * fin + exp2f(sink2 - mf);
    }
    fin *= ll > 0.f ? 1.0f / ll : 0.f;
    const bool wide = ex.gate != nullptr && ex.gate_wide > 0;
    if (ex.gate != nullptr && !wide) fin *= 1.0f / (1.0f + expf(-__bfloat162float(((const bf16*)ex.gate)[(int64_t)row * ex.gate_ld + head])));
    const bf16* gw = (const bf16*)ex.gate + (int64_t)row * ex.gate_ld + (int64_t)head * sh.vd;
    const int64_t orow = ((int64_t)row * q_heads + head) * sh.vd;
    for (int c = c0; c < sh.vd; c += 8) {
        float acc = 0.f;
        for (int w = 0; w < 4; ++w) acc += mg[((int64_t)w * 16 + item) * ps + 2 + c] * f[w];
        acc *= fin;
        if (wide) acc *= 1.0f / (1.0f + expf(-__bfloat162float(gw[c])));
        fx_store(out, orow + c, acc, ex.out_f32 > 0);
    }
}

// Merges the splits of every unit in split order and writes the rows out.  One block of 256 threads per
// unit.  First a warp per item (q head) reads the splits' maxima and sums, one split per lane, and leaves
// the splits' weights 2^(m_s - m) and the item's final factor (1 / sum, sink, gate) in shared memory; then
// the threads share the (item, column) pairs and add the splits up in split order.
#define FX_MAX_SPLITS 64
__global__ void __launch_bounds__(256)
flex_decode_merge_kernel(const float* __restrict__ scratch, bf16* __restrict__ out, int q_heads, int kv_heads,
                         AttnExtra ex, int vd, int vdp, int chunks, int splits) {
    __shared__ float wgt[16][FX_MAX_SPLITS];
    __shared__ float fin_s[16];
    pdl_prologue();
    const int unit = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = q_heads / kv_heads;
    const int chunk_i = unit % chunks, kh = (unit / chunks) % kv_heads, row = unit / (chunks * kv_heads);
    const int head0 = kh * group + chunk_i * 16, n_items = min(16, group - chunk_i * 16);
    const int ps = vdp + 2;
    const float* base = scratch + (int64_t)unit * splits * 16 * ps;
    const int64_t step = (int64_t)16 * ps;
    for (int item = warp; item < n_items; item += 8) {
        const float* src = base + (int64_t)item * ps;
        const int s0 = lane, s1 = lane + 32;
        const float m0 = s0 < splits ? src[s0 * step] : -INFINITY, m1 = s1 < splits ? src[s1 * step] : -INFINITY;
        const float l0 = s0 < splits ? src[s0 * step + 1] : 0.f, l1 = s1 < splits ? src[s1 * step + 1] : 0.f;
        const float mm = warp_max(fmaxf(m0, m1));
        const float ref = mm == -INFINITY ? 0.f : mm;
        const float f0 = exp2f(m0 - ref), f1 = exp2f(m1 - ref);
        if (s0 < splits) wgt[item][s0] = f0;
        if (s1 < splits) wgt[item][s1] = f1;
        float ll = warp_sum(l0 * f0 + l1 * f1);      // (a fixed tree over the lanes: the same bits on every call)
        if (lane == 0) {
            const int head = head0 + item;
            float fin = 1.f;
            if (ex.sink != nullptr) {
                const float sink2 = ex.sink[head] * FX_LOG2E;
                const float mf = fmaxf(mm, sink2);
                fin = exp2f(mm - mf);
                ll = ll * fin + exp2f(sink2 - mf);
            }
            fin *= ll > 0.f ? 1.0f / ll : 0.f;
            if (ex.gate != nullptr && ex.gate_wide <= 0)
                fin *= 1.0f / (1.0f + expf(-__bfloat162float(((const bf16*)ex.gate)[(int64_t)row * ex.gate_ld + head])));
            fin_s[item] = fin;
        }
    }
    __syncthreads();
    const int64_t orow = ((int64_t)row * q_heads + head0) * vd;
    for (int i = tid; i < n_items * vd; i += 256) {
        const int item = i / vd, c = i - item * vd;
        const float* src = base + (int64_t)item * ps + 2 + c;
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) acc += src[s * step] * wgt[item][s];
        acc *= fin_s[item];
        if (ex.gate != nullptr && ex.gate_wide > 0)      // heads head0 .. of the row lie one after the other: value i of them
            acc *= 1.0f / (1.0f + expf(-__bfloat162float(((const bf16*)ex.gate)[(int64_t)row * ex.gate_ld + (int64_t)head0 * vd + i])));
        fx_store(out, orow + i, acc, ex.out_f32 > 0);
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
// The value widths the kernels are compiled for: the accumulators of a thread are a template size.
static int fx_value_bucket(int vd) {
    const int buckets[] = {16, 32, 48, 64, 96, 128, 192, 256};
    for (int b : buckets)
        if (vd <= b) return b;
    return 0;
}

static void fx_fill_shape(int dk, int vd, bool v_from_k, FxShape* sh) {
    sh->dk = dk;
    sh->vd = vd;
    sh->dkp = (dk + 15) / 16 * 16;
    sh->vdp = fx_value_bucket(vd);
    // a value tile row is read up to the bucket's width: where the values are the head of the key rows,
    // the key rows are that long at least (what lies past the real width feeds columns that are never stored)
    sh->ks = (v_from_k && sh->vdp > sh->dkp ? sh->vdp : sh->dkp) + 8;
    sh->vs = sh->vdp + 8;
}

static int fx_shape(const PagedCache& cache, const AttnExtra& ex, FxShape* sh) {
    fx_fill_shape(cache.head_dim, ex.v_from_k > 0 ? ex.v_from_k : cache_v_dim(cache), ex.v_from_k > 0, sh);
    X0NE_REQUIRE(cache.page_size == FX_PAGE, "attention_flex: pages of %d positions, the kernel takes %d", cache.page_size, FX_PAGE);
    X0NE_REQUIRE(sh->dk > 0 && sh->vd > 0 && sh->vdp > 0, "attention_flex: values of %d are beyond the kernel's 256", sh->vd);
    X0NE_REQUIRE(ex.v_from_k <= cache.head_dim, "attention_flex: values of %d out of keys of %d", ex.v_from_k, cache.head_dim);
    X0NE_REQUIRE(ex.v_from_k > 0 || cache.v_dim >= 0, "attention_flex: the cache keeps no values");
    return 0;
}

static size_t fx_prefill_smem(const FxShape& sh, bool v_from_k) {
    return ((size_t)(FX_TILE_ROWS + 2 * FX_PAGE) * sh.ks + (v_from_k ? 0 : (size_t)2 * FX_PAGE * sh.vs)) * sizeof(bf16);
}
static size_t fx_decode_smem(const FxShape& sh, bool v_from_k) {
    const size_t tiles = FX_DECODE_STAGES * ((size_t)FX_PAGE * sh.ks + (v_from_k ? 0 : (size_t)FX_PAGE * sh.vs)) * sizeof(bf16);
    const size_t merge = (size_t)4 * 16 * (sh.vdp + 2) * sizeof(float);
    return (size_t)16 * sh.ks * sizeof(bf16) + (tiles > merge ? tiles : merge);
}

X0NE_API int x0ne_attention_flex_tile_rows() { return FX_TILE_ROWS; }

// Shared memory the kernels need for a shape (prefill, decode), for the caller's routing; 0 = not taken.
X0NE_API int64_t x0ne_attention_flex_smem(int dk, int vd, int v_from_k, int decode) {
    FxShape sh;
    if (dk <= 0 || (v_from_k > 0 ? v_from_k : vd) <= 0) return 0;
    fx_fill_shape(dk, v_from_k > 0 ? v_from_k : vd, v_from_k > 0, &sh);
    if (sh.vdp == 0) return 0;
    return (int64_t)(decode ? fx_decode_smem(sh, v_from_k > 0) : fx_prefill_smem(sh, v_from_k > 0));
}

template <typename K>
static int fx_allow_smem(K kernel, size_t smem) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        X0NE_REQUIRE(e == cudaSuccess, "attention_flex: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    return 0;
}

X0NE_API int x0ne_attention_flex_prefill(const void* q, void* out, PagedCache cache, const int32_t* tile_seq,
                                         const int32_t* tile_row0, int n_tiles, const int32_t* seq_first_row,
                                         const int32_t* seq_slot, const int32_t* seq_pos0, int q_heads, float scale, int window,
                                         AttnExtra ex, cudaStream_t stream) {
    X0NE_REQUIRE(n_tiles >= 0 && q_heads > 0 && cache.kv_heads > 0 && q_heads % cache.kv_heads == 0 && q_heads <= 65535,
                 "attention_flex: %d q heads over %d kv heads", q_heads, cache.kv_heads);
    X0NE_REQUIRE(window >= 0 && ex.chunk >= 0 && ex.keep_first >= 0, "attention_flex: negative window, chunk or count of kept keys");
    FxShape sh;
    if (int e = fx_shape(cache, ex, &sh)) return e;
    if (n_tiles == 0) return 0;
    const size_t smem = fx_prefill_smem(sh, ex.v_from_k > 0);
    X0NE_REQUIRE(smem <= 227 * 1024, "attention_flex: keys of %d need %zu bytes of shared memory", sh.dk, smem);
    const dim3 grid(n_tiles, q_heads), block(256);
#define FX_PREFILL(DVT)                                                                                                     \
    do {                                                                                                                    \
        if (int e = fx_allow_smem(flex_prefill_kernel<DVT>, smem)) return e;                                                \
        x0ne_launch(flex_prefill_kernel<DVT>, grid, block, smem, stream, (const bf16*)q, (bf16*)out, cache, tile_seq, tile_row0, \
                    seq_first_row, seq_slot, seq_pos0, q_heads, scale, window, ex, sh);                                     \
    } while (0)
    switch (sh.vdp) {
        case 16: FX_PREFILL(2); break;
        case 32: FX_PREFILL(4); break;
        case 48: FX_PREFILL(6); break;
        case 64: FX_PREFILL(8); break;
        case 96: FX_PREFILL(12); break;
        case 128: FX_PREFILL(16); break;
        case 192: FX_PREFILL(24); break;
        default: FX_PREFILL(32); break;
    }
#undef FX_PREFILL
    X0NE_LAUNCH_CHECK();
}

X0NE_API int64_t x0ne_attention_flex_scratch_bytes(int n_rows, int q_heads, int kv_heads, int vd, int splits) {
    const int chunks = (q_heads / kv_heads + 15) / 16, vdp = fx_value_bucket(vd);
    return splits > 1 ? (int64_t)n_rows * kv_heads * chunks * splits * 16 * (vdp + 2) * (int64_t)sizeof(float) : 0;
}

X0NE_API int x0ne_attention_flex_decode(const void* q, void* out, PagedCache cache, const int32_t* row_slot,
                                        const int32_t* row_pos, int n_rows, int q_heads, float scale, int window, AttnExtra ex,
                                        int splits, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && q_heads > 0 && cache.kv_heads > 0 && q_heads % cache.kv_heads == 0,
                 "attention_flex: %d q heads over %d kv heads", q_heads, cache.kv_heads);
    X0NE_REQUIRE(window >= 0 && ex.chunk >= 0 && ex.keep_first >= 0 && splits >= 1 && splits <= FX_MAX_SPLITS, "attention_flex: window, chunk or splits (1 to %d) out of range", FX_MAX_SPLITS);
    FxShape sh;
    if (int e = fx_shape(cache, ex, &sh)) return e;
    if (n_rows == 0) return 0;
    const int chunks = (q_heads / cache.kv_heads + 15) / 16;
    const int64_t units = (int64_t)n_rows * cache.kv_heads * chunks;
    X0NE_REQUIRE(units <= 0x7fffffff, "attention_flex: too many rows");
    X0NE_REQUIRE(splits == 1 || (scratch != nullptr && scratch_bytes >= x0ne_attention_flex_scratch_bytes(n_rows, q_heads, cache.kv_heads, sh.vd, splits)),
                 "attention_flex: %d splits need %lld bytes of scratch", splits,
                 (long long)x0ne_attention_flex_scratch_bytes(n_rows, q_heads, cache.kv_heads, sh.vd, splits));
    const size_t smem = fx_decode_smem(sh, ex.v_from_k > 0);
    X0NE_REQUIRE(smem <= 227 * 1024, "attention_flex: keys of %d need %zu bytes of shared memory", sh.dk, smem);
    const dim3 grid((unsigned)units, splits), block(128);
#define FX_DECODE(DVT)                                                                                                       \
    do {                                                                                                                     \
        if (int e = fx_allow_smem(flex_decode_kernel<DVT>, smem)) return e;                                                  \
        x0ne_launch(flex_decode_kernel<DVT>, grid, block, smem, stream, (const bf16*)q, (bf16*)out, cache, row_slot, row_pos, q_heads, \
                    scale, window, ex, sh, chunks, splits, (float*)scratch);                                                 \
    } while (0)
    switch (sh.vdp) {
        case 16: FX_DECODE(2); break;
        case 32: FX_DECODE(4); break;
        case 48: FX_DECODE(6); break;
        case 64: FX_DECODE(8); break;
        case 96: FX_DECODE(12); break;
        case 128: FX_DECODE(16); break;
        case 192: FX_DECODE(24); break;
        default: FX_DECODE(32); break;
    }
#undef FX_DECODE
    if (splits > 1) {
        cudaError_t e = cudaGetLastError();
        X0NE_REQUIRE(e == cudaSuccess, "attention_flex: %s", cudaGetErrorString(e));
        x0ne_launch(flex_decode_merge_kernel, dim3((unsigned)units), dim3(256), 0, stream, (const float*)scratch, (bf16*)out, q_heads,
                    cache.kv_heads, ex, sh.vd, sh.vdp, chunks, splits);
    }
    X0NE_LAUNCH_CHECK();
}
