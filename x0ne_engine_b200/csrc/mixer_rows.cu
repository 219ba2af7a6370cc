// Row-wise kernels of mixers and feed-forwards beyond the pre-norm GQA block: a clipped gated
// activation, the cache write of an attention whose values are blended with an earlier layer's,
// and the preparation of a latent attention's queries and cache rows (latent norm, interleaved
// rotary pairs with a per-pair frequency table).  Templated on the activation type like the
// kernels of elementwise.cu; per-channel weights, angles, norms and blends are float32.
#include "common.cuh"

// ----------------------------------------------------------------------------------------
// Clipped gated activation on the packed [gate; up] row:
//   g = min(gate, limit); u = clamp(up, -limit, limit); out = g * sigmoid(slope * g) * (u + shift)
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void glu_clipped_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int64_t total, float limit,
                                   float slope, float shift) {
    pdl_prologue();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / inter;
        const int col = (int)(i % inter);
        const float g = fminf(to_f32(gate_up[row * 2 * inter + col]), limit);
        const float u = fminf(fmaxf(to_f32(gate_up[row * 2 * inter + inter + col]), -limit), limit);
        out[i] = from_f32<T>(g / (1.0f + expf(-slope * g)) * (u + shift));
    }
}

// 8 values per thread with 16-byte accesses (inter % 8 == 0 and aligned rows).
template <typename T>
__global__ void glu_clipped_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int64_t total8, float limit,
                                       float slope, float shift) {
    pdl_prologue();
    const int per_row = inter / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / per_row;
        const int col = (int)(i % per_row) * 8;
        const T* g = gate_up + row * 2 * inter + col;
        T gv[8], uv[8], ov[8];
        if (sizeof(T) == 2) {
            *reinterpret_cast<uint4*>(gv) = *reinterpret_cast<const uint4*>(g);
            *reinterpret_cast<uint4*>(uv) = *reinterpret_cast<const uint4*>(g + inter);
        } else {
            reinterpret_cast<uint4*>(gv)[0] = reinterpret_cast<const uint4*>(g)[0];
            reinterpret_cast<uint4*>(gv)[1] = reinterpret_cast<const uint4*>(g)[1];
            reinterpret_cast<uint4*>(uv)[0] = reinterpret_cast<const uint4*>(g + inter)[0];
            reinterpret_cast<uint4*>(uv)[1] = reinterpret_cast<const uint4*>(g + inter)[1];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float a = fminf(to_f32(gv[k]), limit);
            const float u = fminf(fmaxf(to_f32(uv[k]), -limit), limit);
            ov[k] = from_f32<T>(a / (1.0f + expf(-slope * a)) * (u + shift));
        }
        T* o = out + row * inter + col;
        if (sizeof(T) == 2) {
            *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(ov);
        } else {
            reinterpret_cast<uint4*>(o)[0] = reinterpret_cast<const uint4*>(ov)[0];
            reinterpret_cast<uint4*>(o)[1] = reinterpret_cast<const uint4*>(ov)[1];
        }
    }
}

X0NE_API int x0ne_glu_clipped(const void* gate_up, void* out, int dt, int n_rows, int inter, float limit, float slope,
                              float shift, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && inter > 0 && limit > 0.f, "glu_clipped: rows %d width %d limit %g", n_rows, inter, limit);
    if (n_rows == 0) return 0;
    const int64_t total = (int64_t)n_rows * inter;
    if (inter % 8 == 0 && ((((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) && (dt == X0NE_F32 || dt == X0NE_BF16)) {
        const int64_t total8 = total / 8;
        const unsigned grid8 = (unsigned)((total8 + 255) / 256 < 65535 * 16 ? (total8 + 255) / 256 : 65535 * 16);
        if (dt == X0NE_F32)
            x0ne_launch(glu_clipped_vec_kernel<float>, dim3(grid8), dim3(256), 0, stream, (const float*)gate_up, (float*)out, inter, total8, limit, slope, shift);
        else
            x0ne_launch(glu_clipped_vec_kernel<bf16>, dim3(grid8), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total8, limit, slope, shift);
        X0NE_LAUNCH_CHECK();
    }
    const unsigned grid = (unsigned)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
    if (dt == X0NE_F32)
        x0ne_launch(glu_clipped_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)gate_up, (float*)out, inter, total, limit, slope, shift);
    else if (dt == X0NE_BF16)
        x0ne_launch(glu_clipped_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total, limit, slope, shift);
    else
        X0NE_REQUIRE(false, "glu_clipped: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// 8 consecutive values as 16-byte (bfloat16) or 2 x 16-byte (float) accesses
__device__ __forceinline__ void copy8(bf16* d, const bf16* s) { *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s); }
__device__ __forceinline__ void copy8(float* d, const float* s) {
    reinterpret_cast<float4*>(d)[0] = reinterpret_cast<const float4*>(s)[0];
    reinterpret_cast<float4*>(d)[1] = reinterpret_cast<const float4*>(s)[1];
}
__device__ __forceinline__ void load8f(const bf16* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8f(const float* p, float* v) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8f(bf16* p, const float* v) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void store8f(float* p, const float* v) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}

// ----------------------------------------------------------------------------------------
// K/V write of an attention without rotation.  `src` holds, per row of `ld` values, the keys at
// column k_col (kv_heads x k_dim) and the values at column v_col (kv_heads x v_dim).
//   mode 0: keys and values go to the cache as they are.
//   mode 1: the same, and the values are also kept in `v_first` (rows of kv_heads x v_dim) for
//           the later layers of this pass.
//   mode 2: v = (1 - lambda) v + lambda v_first[row] in float32, lambda read from the device.
// One block per row; a row whose position has no page (or whose slot is negative) writes nothing
// into the cache.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void kv_write_blend_kernel(const T* __restrict__ src, int ld, int k_col, int v_col, T* __restrict__ v_first,
                                      const float* __restrict__ lambda, int mode, PagedCache cache,
                                      const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos, int vec) {
    pdl_launch_dependents();
    const float lam = mode == 2 ? lambda[0] : 0.f;
    const int row = blockIdx.x;
    const int slot = row_slot[row], pos = row_pos[row];
    pdl_wait();
    const int kd = cache.head_dim, vd = cache_v_dim(cache), kvh = cache.kv_heads;
    T* base = (T*)cache.base;
    const T* s = src + (int64_t)row * ld;
    const int64_t k0 = cache_row_offset(cache, slot, pos, 0, 0);
    const int64_t head_k = (int64_t)cache.page_size * kd, head_v = (int64_t)cache.page_size * vd;
    if (vec) {
        // 8 values at a time (16 bytes of bfloat16): every width and column is a multiple of 8 and the rows are aligned
        const int64_t v0 = cache_row_offset(cache, slot, pos, 0, 1);
        const int nk = kvh * kd / 8, nv = kvh * vd / 8;
        for (int i = threadIdx.x; i < nk + nv; i += blockDim.x) {
            if (i < nk) {
                const int e = i * 8;
                if (k0 >= 0) copy8(base + k0 + (e / kd) * head_k + (e % kd), s + k_col + e);
                continue;
            }
            const int e = (i - nk) * 8;
            float v[8];
            load8f(s + v_col + e, v);
            T* first = v_first + (int64_t)row * kvh * vd + e;
            if (mode == 1) copy8(first, s + v_col + e);
            if (mode == 2) {
                float f[8];
                load8f(first, f);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = (1.0f - lam) * v[k] + lam * f[k];
            }
            if (v0 >= 0) store8f(base + v0 + (e / vd) * head_v + (e % vd), v);
        }
        return;
    }
    if (k0 >= 0)
        for (int i = threadIdx.x; i < kvh * kd; i += blockDim.x) base[k0 + (i / kd) * head_k + (i % kd)] = s[k_col + i];
    const int64_t v0 = cache_row_offset(cache, slot, pos, 0, 1);
    for (int i = threadIdx.x; i < kvh * vd; i += blockDim.x) {
        T v = s[v_col + i];
        if (mode == 1) v_first[(int64_t)row * kvh * vd + i] = v;
        if (mode == 2) v = from_f32<T>((1.0f - lam) * to_f32(v) + lam * to_f32(v_first[(int64_t)row * kvh * vd + i]));
        if (v0 >= 0) base[v0 + (i / vd) * head_v + (i % vd)] = v;
    }
}

X0NE_API int x0ne_kv_write_blend(const void* src, int dt, int ld, int k_col, int v_col, void* v_first, const float* lambda,
                                 int mode, PagedCache cache, const int32_t* row_slot, const int32_t* row_pos, int n_rows,
                                 cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && ld > 0 && k_col >= 0 && v_col >= 0 && mode >= 0 && mode <= 2, "kv_write: rows %d ld %d mode %d", n_rows, ld, mode);
    X0NE_REQUIRE(cache.v_dim >= 0, "kv_write: the cache keeps no values");
    X0NE_REQUIRE(k_col + cache.kv_heads * cache.head_dim <= ld && v_col + cache.kv_heads * cache_v_dim(cache) <= ld,
                 "kv_write: keys or values lie outside the source rows");
    X0NE_REQUIRE(mode == 0 || v_first != nullptr, "kv_write: mode %d needs the buffer of first values", mode);
    X0NE_REQUIRE(mode != 2 || lambda != nullptr, "kv_write: blending needs its weight");
    if (n_rows == 0) return 0;
    const int vd = cache_v_dim(cache);
    const int vec = (cache.head_dim % 8 == 0 && vd % 8 == 0 && ld % 8 == 0 && k_col % 8 == 0 && v_col % 8 == 0 &&
                     ((((uintptr_t)src | (uintptr_t)v_first | (uintptr_t)cache.base) & 31) == 0) && cache.page_stride % 8 == 0) ? 1 : 0;
    if (dt == X0NE_F32)
        x0ne_launch(kv_write_blend_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (const float*)src, ld, k_col, v_col, (float*)v_first, lambda, mode, cache, row_slot, row_pos, vec);
    else if (dt == X0NE_BF16)
        x0ne_launch(kv_write_blend_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, (const bf16*)src, ld, k_col, v_col, (bf16*)v_first, lambda, mode, cache, row_slot, row_pos, vec);
    else
        X0NE_REQUIRE(false, "kv_write: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Latent attention, preparation of a pass's rows.  `src` holds per row of `ld` values the queries
// at column 0 (heads x (dim + rot)) and, at column dkv_col, `rank` latent values followed by `rot`
// values of the key part that all heads share.
//   c = latent * rsqrt(mean(latent^2) + eps) * w        -> cache row [0, rank)
//   shared key part, rotated                             -> cache row [rank, rank + rot)
//   q_out[row][head] = [ q_abs[head][row][0..rank) , rotated q[row][head][dim..dim+rot) ]
// where q_abs (heads x rows_stride x rank) holds each head's unrotated query already multiplied
// into the latent space, so that a score is one dot product of rank + rot values with the cache
// row.  Rotation: pair (2i, 2i+1) turns by pos * freq[i]; cos and sin are scaled by `mag`.
// `table` (float32 [positions][rot]: rot/2 cosines then rot/2 sines, already scaled) replaces the
// computation for the positions it covers.  One block per row.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ src, int ld, int dkv_col, const T* __restrict__ q_abs,
                                      int64_t q_abs_head_stride, const float* __restrict__ norm_w, float eps,
                                      const float* __restrict__ freq, float mag, const float* __restrict__ table,
                                      int table_positions, T* __restrict__ q_out, int heads, int dim, int rot, int rank,
                                      PagedCache cache, const int32_t* __restrict__ row_slot,
                                      const int32_t* __restrict__ row_pos, int write_cache) {
    extern __shared__ float cs[];          // rot/2 cosines, rot/2 sines
    __shared__ float partial[32];
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int slot = row_slot[row], pos = row_pos[row];
    const int half = rot / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        if (pos >= 0 && pos < table_positions) {
            cs[i] = table[(int64_t)pos * rot + i];
            cs[half + i] = table[(int64_t)pos * rot + half + i];
        } else {
            float sn, c;
            sincosf((float)pos * freq[i], &sn, &c);
            cs[i] = c * mag;
            cs[half + i] = sn * mag;
        }
    }
    pdl_wait();
    const T* s = src + (int64_t)row * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f32(s[dkv_col + i]);
        ss = fmaf(v, v, ss);
    }
    const float scale = 1.0f / sqrtf(block_reduce(ss, partial, OpSum(), 0.f) / (float)rank + eps);   // (syncs: cs is complete)
    const int64_t k0 = write_cache ? cache_row_offset(cache, slot, pos, 0, 0) : -1;
    if (k0 >= 0) {
        T* kr = (T*)cache.base + k0;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) kr[i] = from_f32<T>(to_f32(s[dkv_col + i]) * scale * norm_w[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = to_f32(s[dkv_col + rank + 2 * i]), v = to_f32(s[dkv_col + rank + 2 * i + 1]);
            kr[rank + 2 * i] = from_f32<T>(u * cs[i] - v * cs[half + i]);
            kr[rank + 2 * i + 1] = from_f32<T>(v * cs[i] + u * cs[half + i]);
        }
    }
    const int qw = rank + rot;
    T* qo = q_out + (int64_t)row * heads * qw;
    if (rank % 8 == 0 && qw % 8 == 0 && q_abs_head_stride % 8 == 0 && ((((uintptr_t)q_out | (uintptr_t)q_abs) & 31) == 0)) {
        const int per_head = rank / 8;
        for (int i = threadIdx.x; i < heads * per_head; i += blockDim.x) {
            const int h = i / per_head, d = (i - h * per_head) * 8;
            copy8(qo + h * qw + d, q_abs + h * q_abs_head_stride + (int64_t)row * rank + d);
        }
    } else {
        for (int i = threadIdx.x; i < heads * rank; i += blockDim.x) {
            const int h = i / rank, d = i % rank;
            qo[h * qw + d] = q_abs[h * q_abs_head_stride + (int64_t)row * rank + d];
        }
    }
    for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        const T* qr = s + h * (dim + rot) + dim;
        const float u = to_f32(qr[2 * j]), v = to_f32(qr[2 * j + 1]);
        qo[h * qw + rank + 2 * j] = from_f32<T>(u * cs[j] - v * cs[half + j]);
        qo[h * qw + rank + 2 * j + 1] = from_f32<T>(v * cs[j] + u * cs[half + j]);
    }
}

X0NE_API int x0ne_latent_prepare(const void* src, int dt, int ld, int dkv_col, const void* q_abs, int64_t q_abs_head_stride,
                                 const float* norm_w, float eps, const float* freq, float mag, const float* table,
                                 int table_positions, void* q_out, int heads, int dim, int rot, int rank, PagedCache cache,
                                 const int32_t* row_slot, const int32_t* row_pos, int n_rows, int write_cache,
                                 cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && heads > 0 && dim > 0 && rot >= 0 && rot % 2 == 0 && rank > 0, "latent_prepare: heads %d dim %d rot %d rank %d", heads, dim, rot, rank);
    X0NE_REQUIRE(cache.kv_heads == 1 && cache.head_dim == rank + rot, "latent_prepare: the cache row is %d x %d, not 1 x %d", cache.kv_heads, cache.head_dim, rank + rot);
    X0NE_REQUIRE(heads * (dim + rot) <= dkv_col && dkv_col + rank + rot <= ld, "latent_prepare: columns lie outside the source rows");
    X0NE_REQUIRE(rot == 0 || freq != nullptr, "latent_prepare: no frequencies");
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
    if (dt == X0NE_F32)
        x0ne_launch(latent_prepare_kernel<float>, dim3(n_rows), dim3(256), smem, stream, (const float*)src, ld, dkv_col, (const float*)q_abs, q_abs_head_stride, norm_w, eps, freq, mag, table, table_positions, (float*)q_out, heads, dim, rot, rank, cache, row_slot, row_pos, write_cache);
    else if (dt == X0NE_BF16)
        x0ne_launch(latent_prepare_kernel<bf16>, dim3(n_rows), dim3(256), smem, stream, (const bf16*)src, ld, dkv_col, (const bf16*)q_abs, q_abs_head_stride, norm_w, eps, freq, mag, table, table_positions, (bf16*)q_out, heads, dim, rot, rank, cache, row_slot, row_pos, write_cache);
    else
        X0NE_REQUIRE(false, "latent_prepare: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Attention rows whose queries and keys are normed over the WHOLE projection (all heads at once,
// one weight per projected value) before they are split into heads and rotated:
//   q_n = q * rsqrt(mean(q^2 over q_heads x dim) + eps) * w_q      (k alike, over kv_heads x dim)
//   rotation of the first `rot` values of every head, value i with value i + rot/2, by pos * freq[i]
//   q_n -> q_out; k_n -> cache keys; v -> cache values (as they are).
// `src` rows of `ld` values hold the queries at column 0, the keys at k_col and the values at v_col.
// write_kv == 0: a layer that reads another layer's keys and values; only the queries are made.
// Norms, angles and the rotation are float32; one rounding at the store.  One block per row.
// `table` (float32 [positions][rot]: rot/2 cosines then rot/2 sines) replaces sincosf for the
// positions it covers.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void whole_norm_rope_kv_write_kernel(const T* __restrict__ src, int ld, int k_col, int v_col,
                                                const float* __restrict__ norm_q, const float* __restrict__ norm_k, float eps,
                                                const float* __restrict__ freq, int rot, const float* __restrict__ table,
                                                int table_positions, T* __restrict__ q_out, int q_heads, PagedCache cache,
                                                const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                                int write_kv) {
    extern __shared__ float cs[];          // rot/2 cosines, rot/2 sines
    __shared__ float partial[32];
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int slot = row_slot[row], pos = row_pos[row];
    const int half = rot / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        if (pos >= 0 && pos < table_positions) {
            cs[i] = table[(int64_t)pos * rot + i];
            cs[half + i] = table[(int64_t)pos * rot + half + i];
        } else {
            float sn, c;
            sincosf((float)pos * freq[i], &sn, &c);
            cs[i] = c;
            cs[half + i] = sn;
        }
    }
    pdl_wait();
    const int D = cache.head_dim, G = cache.kv_heads, vd = cache_v_dim(cache);
    const int qn = q_heads * D, kn = G * D;
    const T* s = src + (int64_t)row * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < qn; i += blockDim.x) {
        const float v = to_f32(s[i]);
        sq = fmaf(v, v, sq);
    }
    if (write_kv)
        for (int i = threadIdx.x; i < kn; i += blockDim.x) {
            const float v = to_f32(s[k_col + i]);
            sk = fmaf(v, v, sk);
        }
    const float scale_q = 1.0f / sqrtf(block_reduce(sq, partial, OpSum(), 0.f) / (float)qn + eps);   // (syncs: cs is complete)
    T* qo = q_out + (int64_t)row * qn;
    for (int i = threadIdx.x; i < qn; i += blockDim.x) {
        const int d = i % D;
        float a = to_f32(s[i]) * scale_q * norm_q[i];
        if (d < rot) {
            const int j = d < half ? d : d - half;
            const int ip = d < half ? i + half : i - half;
            const float b = to_f32(s[ip]) * scale_q * norm_q[ip];
            a = d < half ? a * cs[j] - b * cs[half + j] : a * cs[j] + b * cs[half + j];
        }
        qo[i] = from_f32<T>(a);
    }
    if (!write_kv) return;
    const float scale_k = 1.0f / sqrtf(block_reduce(sk, partial, OpSum(), 0.f) / (float)kn + eps);
    const int64_t k0 = cache_row_offset(cache, slot, pos, 0, 0);
    if (k0 < 0) return;
    T* base = (T*)cache.base;
    const int64_t head_k = (int64_t)cache.page_size * D, head_v = (int64_t)cache.page_size * vd;
    for (int i = threadIdx.x; i < kn; i += blockDim.x) {
        const int d = i % D;
        float a = to_f32(s[k_col + i]) * scale_k * norm_k[i];
        if (d < rot) {
            const int j = d < half ? d : d - half;
            const int ip = d < half ? i + half : i - half;
            const float b = to_f32(s[k_col + ip]) * scale_k * norm_k[ip];
            a = d < half ? a * cs[j] - b * cs[half + j] : a * cs[j] + b * cs[half + j];
        }
        base[k0 + (i / D) * head_k + d] = from_f32<T>(a);
    }
    const int64_t v0 = cache_row_offset(cache, slot, pos, 0, 1);
    for (int i = threadIdx.x; i < G * vd; i += blockDim.x) base[v0 + (i / vd) * head_v + (i % vd)] = s[v_col + i];
}

// The same with 16-byte accesses: every width, column and half of the rotated part a multiple of 8.  A thread takes
// pieces of 8 consecutive values; a rotated piece reads its partner piece (8 values rot/2 further on or back).
template <typename T>
__device__ __forceinline__ void wn_rotated_piece(const T* __restrict__ s, const float* __restrict__ w, int i, int D, int rot, int half,
                                                 float scale, const float* __restrict__ cs, float* a) {
    float wa[8];
    load8f(s + i, a);
    load8f(w + i, wa);
    const int d = i % D;
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = a[k] * scale * wa[k];
    if (d < rot) {
        const bool lo = d < half;
        const int ip = lo ? i + half : i - half, j = lo ? d : d - half;
        float b[8], wb[8];
        load8f(s + ip, b);
        load8f(w + ip, wb);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float bk = b[k] * scale * wb[k];
            a[k] = lo ? a[k] * cs[j + k] - bk * cs[half + j + k] : a[k] * cs[j + k] + bk * cs[half + j + k];
        }
    }
}

// STAGE: a thread keeps its pieces of the row's queries and keys (at most WN_MAX_PIECES of 8 values) and their norm
// weights in registers from the one read of global memory; the two sums of squares meet in one exchange through shared
// memory; the normed values are parked in shared memory as float32, from where the rotation reads a piece's partner.
// Without STAGE (rows too long for that) the rotation reads global memory again.
#define WN_MAX_PIECES 4
template <typename T, bool STAGE>
__global__ void __launch_bounds__(256) whole_norm_rope_kv_write_vec_kernel(
    const T* __restrict__ src, int ld, int k_col, int v_col, const float* __restrict__ norm_q, const float* __restrict__ norm_k,
    float eps, const float* __restrict__ freq, int rot, const float* __restrict__ table, int table_positions, T* __restrict__ q_out,
    int q_heads, PagedCache cache, const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos, int write_kv) {
    extern __shared__ float cs[];
    __shared__ float partial[32];
    __shared__ float partial2[64];
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int slot = row_slot[row], pos = row_pos[row];
    const int half = rot / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        if (pos >= 0 && pos < table_positions) {
            cs[i] = table[(int64_t)pos * rot + i];
            cs[half + i] = table[(int64_t)pos * rot + half + i];
        } else {
            float sn, c;
            sincosf((float)pos * freq[i], &sn, &c);
            cs[i] = c;
            cs[half + i] = sn;
        }
    }
    const int D = cache.head_dim, G = cache.kv_heads, vd = cache_v_dim(cache);
    const int qn = q_heads * D, kn = write_kv ? G * D : 0, vn = write_kv ? G * vd : 0;
    const int64_t k0 = write_kv ? cache_row_offset(cache, slot, pos, 0, 0) : -1;       // (page numbers are older than any running kernel)
    const int64_t v0 = write_kv ? cache_row_offset(cache, slot, pos, 0, 1) : -1;
    T* qo = q_out + (int64_t)row * qn;
    T* base = (T*)cache.base;
    const int64_t head_k = (int64_t)cache.page_size * D, head_v = (int64_t)cache.page_size * vd;
    float* stage = cs + (rot > 8 ? rot : 8);          // [qn + kn] when STAGE
    if (STAGE) {
        float v[WN_MAX_PIECES][8], w[WN_MAX_PIECES][8];
#pragma unroll
        for (int u = 0; u < WN_MAX_PIECES; ++u) {                      // (weights are older than any running kernel)
            const int i = (threadIdx.x + u * 256) * 8;
            if (i < qn + kn) load8f(i < qn ? norm_q + i : norm_k + (i - qn), w[u]);
        }
        pdl_wait();
        const T* s = src + (int64_t)row * ld;
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int u = 0; u < WN_MAX_PIECES; ++u) {
            const int i = (threadIdx.x + u * 256) * 8;
            if (i < qn + kn) {
                load8f(i < qn ? s + i : s + k_col + (i - qn), v[u]);
                float ss = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) ss = fmaf(v[u][k], v[u][k], ss);
                if (i < qn) sq += ss; else sk += ss;
            }
        }
        // both sums at once: the warps' sums meet in shared memory and every thread adds them up in warp order
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { partial2[warp] = sq; partial2[32 + warp] = sk; }
        __syncthreads();                                              // (also: cs is complete)
        float tq = 0.f, tk = 0.f;
#pragma unroll
        for (int x = 0; x < 8; ++x) { tq += partial2[x]; tk += partial2[32 + x]; }
        const float scale_q = 1.0f / sqrtf(tq / (float)qn + eps);
        const float scale_k = write_kv ? 1.0f / sqrtf(tk / (float)kn + eps) : 0.f;
#pragma unroll
        for (int u = 0; u < WN_MAX_PIECES; ++u) {
            const int i = (threadIdx.x + u * 256) * 8;
            if (i < qn + kn) {
                const float sc = i < qn ? scale_q : scale_k;
#pragma unroll
                for (int k = 0; k < 8; ++k) v[u][k] = v[u][k] * sc * w[u][k];
                store8f(stage + i, v[u]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < WN_MAX_PIECES; ++u) {
            const int i = (threadIdx.x + u * 256) * 8;
            if (i >= qn + kn) continue;
            const bool is_q = i < qn;
            const int ih = is_q ? i : i - qn;               // index within the q or the k projection
            if (!is_q && k0 < 0) continue;
            const int d = ih % D;
            if (d < rot) {
                const bool lo = d < half;
                const int j = lo ? d : d - half;
                float b[8];
                load8f(stage + (lo ? i + half : i - half), b);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    v[u][k] = lo ? v[u][k] * cs[j + k] - b[k] * cs[half + j + k] : v[u][k] * cs[j + k] + b[k] * cs[half + j + k];
            }
            if (is_q) store8f(qo + i, v[u]);
            else store8f(base + k0 + (ih / D) * head_k + d, v[u]);
        }
        for (int c = threadIdx.x; c < vn / 8; c += blockDim.x) {
            const int iv = c * 8;
            if (v0 >= 0) copy8(base + v0 + (iv / vd) * head_v + iv % vd, s + v_col + iv);
        }
        return;
    }
    pdl_wait();
    const T* s = src + (int64_t)row * ld;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < (qn + kn) / 8; c += blockDim.x) {
        const int i = c * 8;
        float v[8];
        load8f(i < qn ? s + i : s + k_col + (i - qn), v);
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
        if (i < qn) sq += ss; else sk += ss;
    }
    const float scale_q = 1.0f / sqrtf(block_reduce(sq, partial, OpSum(), 0.f) / (float)qn + eps);   // (syncs: cs is complete)
    const float scale_k = write_kv ? 1.0f / sqrtf(block_reduce(sk, partial, OpSum(), 0.f) / (float)kn + eps) : 0.f;
    for (int c = threadIdx.x; c < (qn + kn + vn) / 8; c += blockDim.x) {
        const int i = c * 8;
        float a[8];
        if (i < qn) {
            wn_rotated_piece(s, norm_q, i, D, rot, half, scale_q, cs, a);
            store8f(qo + i, a);
        } else if (i < qn + kn) {
            const int ik = i - qn;
            if (k0 < 0) continue;
            wn_rotated_piece(s + k_col, norm_k, ik, D, rot, half, scale_k, cs, a);
            store8f(base + k0 + (ik / D) * head_k + ik % D, a);
        } else {
            const int iv = i - qn - kn;
            if (v0 >= 0) copy8(base + v0 + (iv / vd) * head_v + iv % vd, s + v_col + iv);
        }
    }
}

X0NE_API int x0ne_whole_norm_rope_kv_write(const void* src, int dt, int ld, int k_col, int v_col, const float* norm_q,
                                           const float* norm_k, float eps, const float* freq, int rot, const float* table,
                                           int table_positions, void* q_out, int q_heads, PagedCache cache,
                                           const int32_t* row_slot, const int32_t* row_pos, int n_rows, int write_kv,
                                           cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && q_heads > 0 && ld >= q_heads * cache.head_dim && rot >= 0 && rot % 2 == 0 && rot <= cache.head_dim,
                 "whole_norm_rope: rows %d heads %d ld %d rot %d head_dim %d", n_rows, q_heads, ld, rot, cache.head_dim);
    X0NE_REQUIRE(norm_q != nullptr && (rot == 0 || freq != nullptr), "whole_norm_rope: no norm weight or no frequencies");
    if (write_kv) {
        X0NE_REQUIRE(cache.v_dim >= 0 && norm_k != nullptr, "whole_norm_rope: the cache keeps no values, or no key norm weight");
        X0NE_REQUIRE(k_col >= q_heads * cache.head_dim && k_col + cache.kv_heads * cache.head_dim <= ld && v_col >= 0 &&
                     v_col + cache.kv_heads * cache_v_dim(cache) <= ld, "whole_norm_rope: keys or values lie outside the source rows");
    }
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
    const int vdw = write_kv ? cache_v_dim(cache) : 8;
    const bool vec = cache.head_dim % 8 == 0 && (rot / 2) % 8 == 0 && ld % 8 == 0 && vdw % 8 == 0 &&
                     (!write_kv || (k_col % 8 == 0 && v_col % 8 == 0 && cache.page_stride % 8 == 0 && (((uintptr_t)cache.base | (uintptr_t)norm_k) & 31) == 0)) &&
                     ((((uintptr_t)src | (uintptr_t)q_out | (uintptr_t)norm_q) & 31) == 0);
    if (vec && (dt == X0NE_F32 || dt == X0NE_BF16)) {
        const size_t head = (size_t)(rot > 8 ? rot : 8) * sizeof(float);
        const size_t staged = head + (size_t)(q_heads + (write_kv ? cache.kv_heads : 0)) * cache.head_dim * sizeof(float);
#define X0NE_WNR(T, STAGE, SMEM) x0ne_launch(whole_norm_rope_kv_write_vec_kernel<T, STAGE>, dim3(n_rows), dim3(256), SMEM, stream, (const T*)src, ld, k_col, v_col, norm_q, norm_k, eps, freq, rot, table, table_positions, (T*)q_out, q_heads, cache, row_slot, row_pos, write_kv)
        // few rows (decode, short prompts): the staged form, which has the shortest path through a row (3.4 against 3.9 us at 8 rows);
        // many rows: the form that keeps few registers and so more rows in flight (98 against 166 us at 8,192 rows)
        // (bfloat16 only: in float32 a row's bits must not depend on how many rows share its pass, and the two forms add in other orders)
        if (dt == X0NE_BF16 && n_rows <= 256 && staged <= 48 * 1024 && (q_heads + (write_kv ? cache.kv_heads : 0)) * cache.head_dim <= WN_MAX_PIECES * 256 * 8) {
            X0NE_WNR(bf16, true, staged);
        } else {
            if (dt == X0NE_F32) X0NE_WNR(float, false, head); else X0NE_WNR(bf16, false, head);
        }
#undef X0NE_WNR
        X0NE_LAUNCH_CHECK();
    }
    if (dt == X0NE_F32)
        x0ne_launch(whole_norm_rope_kv_write_kernel<float>, dim3(n_rows), dim3(256), smem, stream, (const float*)src, ld, k_col, v_col, norm_q, norm_k, eps, freq, rot, table, table_positions, (float*)q_out, q_heads, cache, row_slot, row_pos, write_kv);
    else if (dt == X0NE_BF16)
        x0ne_launch(whole_norm_rope_kv_write_kernel<bf16>, dim3(n_rows), dim3(256), smem, stream, (const bf16*)src, ld, k_col, v_col, norm_q, norm_k, eps, freq, rot, table, table_positions, (bf16*)q_out, q_heads, cache, row_slot, row_pos, write_kv);
    else
        X0NE_REQUIRE(false, "whole_norm_rope: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Squared ReLU in place or out of place: out = max(x, 0)^2, float32 arithmetic.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t total) {
    pdl_prologue();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(x[i]), 0.f);
        out[i] = from_f32<T>(v * v);
    }
}
template <typename T>
__global__ void relu2_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t total8) {
    pdl_prologue();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        float v[8];
        load8f(x + i * 8, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            v[k] = fmaxf(v[k], 0.f);
            v[k] *= v[k];
        }
        store8f(out + i * 8, v);
    }
}

X0NE_API int x0ne_relu2(const void* x, void* out, int dt, int64_t total, cudaStream_t stream) {
    X0NE_REQUIRE(total >= 0 && (dt == X0NE_F32 || dt == X0NE_BF16), "relu2: %lld values, dtype tag %d", (long long)total, dt);
    if (total == 0) return 0;
    if (total % 8 == 0 && ((((uintptr_t)x | (uintptr_t)out) & 31) == 0)) {
        const int64_t t8 = total / 8;
        const unsigned grid = (unsigned)((t8 + 255) / 256 < 65535 * 16 ? (t8 + 255) / 256 : 65535 * 16);
        if (dt == X0NE_F32) x0ne_launch(relu2_vec_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)x, (float*)out, t8);
        else x0ne_launch(relu2_vec_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)x, (bf16*)out, t8);
        X0NE_LAUNCH_CHECK();
    }
    const unsigned grid = (unsigned)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
    if (dt == X0NE_F32) x0ne_launch(relu2_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)x, (float*)out, total);
    else x0ne_launch(relu2_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)x, (bf16*)out, total);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Per-head preparation of an attention without rotation.  src holds, per row, the queries at column 0,
// the keys at k_col and the values at v_col (one packed projection; more columns may follow).
//   query head:  x / sqrt(mean(x^2) + eps) * norm_q[d] * temperature(pos)      -> q_out [rows][q_heads * head_dim]
//                temperature(p) = 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)   (temp_every <= 0: 1)
//   key head:    x / sqrt(mean(x^2) + eps) * norm_k[d]                          -> the row's place in the pages
//   value head:  x / sqrt(mean(x^2) + eps) (v_unit) or x as it is               -> the row's place in the pages
// norm_q / norm_k hold head_dim values shared by all heads (null: no weight).  One warp per (row, head of q, k or v);
// sums of squares, the logarithm and the products are float32.  Rows without a page write no keys or values.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void head_norm_kv_write_kernel(const T* __restrict__ src, int ld, int k_col, int v_col, const float* __restrict__ norm_q,
                                          const float* __restrict__ norm_k, float eps, float temp_coef, int temp_every, int v_unit,
                                          T* __restrict__ q_out, int q_heads, PagedCache cache, const int32_t* __restrict__ row_slot,
                                          const int32_t* __restrict__ row_pos, int n_rows) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int units = q_heads + 2 * cache.kv_heads;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_rows * units) return;
    const int row = (int)(item / units), unit = (int)(item % units);
    const int hd = cache.head_dim, vd = cache_v_dim(cache);
    const int pos = row_pos[row];
    const T* x;
    T* dst;
    const float* w = nullptr;
    int n;
    float mul = 1.f;
    bool normed = true;
    if (unit < q_heads) {
        x = src + (int64_t)row * ld + (int64_t)unit * hd;
        dst = q_out + ((int64_t)row * q_heads + unit) * hd;
        w = norm_q;
        n = hd;
        if (temp_every > 0) mul = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    } else {
        const bool is_k = unit < q_heads + cache.kv_heads;
        const int kh = unit - q_heads - (is_k ? 0 : cache.kv_heads);
        const int64_t off = cache_row_offset(cache, row_slot[row], pos, kh, is_k ? 0 : 1);
        if (off < 0) return;
        n = is_k ? hd : vd;
        x = src + (int64_t)row * ld + (is_k ? k_col : v_col) + (int64_t)kh * n;
        dst = (T*)cache.base + off;
        w = is_k ? norm_k : nullptr;
        normed = is_k || v_unit != 0;
    }
    float scale = mul;
    if (normed) {
        float ss = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float v = to_f32(x[i]);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)n + eps);
    }
    for (int i = lane; i < n; i += 32) {
        float v = to_f32(x[i]) * scale;
        if (w != nullptr) v *= w[i];
        if (normed && mul != 1.f) v *= mul;
        dst[i] = from_f32<T>(v);
    }
}

X0NE_API int x0ne_head_norm_kv_write(const void* src, int dt, int ld, int k_col, int v_col, const float* norm_q, const float* norm_k,
                                     float eps, float temp_coef, int temp_every, int v_unit, void* q_out, int q_heads,
                                     PagedCache cache, const int32_t* row_slot, const int32_t* row_pos, int n_rows,
                                     cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && q_heads > 0 && cache.kv_heads > 0 && cache.head_dim > 0 && cache.v_dim >= 0, "head_norm: bad sizes");
    const int vd = cache_v_dim(cache);
    X0NE_REQUIRE(k_col >= q_heads * cache.head_dim && v_col >= k_col + cache.kv_heads * cache.head_dim && ld >= v_col + cache.kv_heads * vd,
                 "head_norm: columns %d, %d do not fit rows of %d", k_col, v_col, ld);
    if (n_rows == 0) return 0;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * (q_heads + 2 * cache.kv_heads);
    X0NE_REQUIRE((items + warps - 1) / warps <= 0x7fffffff, "head_norm: too many rows");
    const dim3 grid((unsigned)((items + warps - 1) / warps));
    if (dt == X0NE_F32)
        x0ne_launch(head_norm_kv_write_kernel<float>, grid, dim3(warps * 32), 0, stream, (const float*)src, ld, k_col, v_col, norm_q, norm_k,
                    eps, temp_coef, temp_every, v_unit, (float*)q_out, q_heads, cache, row_slot, row_pos, n_rows);
    else if (dt == X0NE_BF16)
        x0ne_launch(head_norm_kv_write_kernel<bf16>, grid, dim3(warps * 32), 0, stream, (const bf16*)src, ld, k_col, v_col, norm_q, norm_k,
                    eps, temp_coef, temp_every, v_unit, (bf16*)q_out, q_heads, cache, row_slot, row_pos, n_rows);
    else
        X0NE_REQUIRE(false, "head_norm: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Bias and activation of a product's rows: out = act(x + bias), float32 inside.
//   act 0: none
//   act 1: a unit with a quadratic positive and an exponential negative branch and the slope 1/2 at zero,
//          z > 0: a z^2 + z / 2;  z <= 0: b (exp(z) - 1 - z) + z / 2      (a, b >= 0 given by the caller)
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const float* __restrict__ bias, T* __restrict__ out, int width, int64_t total,
                                int act, float a, float b) {
    pdl_prologue();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float z = to_f32(x[i]);
        if (bias != nullptr) z += bias[i % width];
        if (act == 1) z = z > 0.f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, expm1f(z) - z, 0.5f * z);
        out[i] = from_f32<T>(z);
    }
}

// the same with 8 values per thread: `width` a multiple of 8 and 16-byte aligned rows
template <typename T>
__global__ void bias_act_vec_kernel(const T* __restrict__ x, const float* __restrict__ bias, T* __restrict__ out, int width, int n_rows,
                                    int act, float a, float b) {
    pdl_launch_dependents();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    float bv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (bias != nullptr) load8f(bias + c, bv);
    pdl_wait();
    for (int row = blockIdx.y; row < n_rows; row += gridDim.y) {
        float z[8];
        load8f(x + (int64_t)row * width + c, z);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            z[i] += bv[i];
            if (act == 1) z[i] = z[i] > 0.f ? fmaf(a * z[i], z[i], 0.5f * z[i]) : fmaf(b, expm1f(z[i]) - z[i], 0.5f * z[i]);
        }
        store8f(out + (int64_t)row * width + c, z);
    }
}

X0NE_API int x0ne_bias_act(const void* x, const float* bias, void* out, int dt, int n_rows, int width, int act, float a, float b,
                           cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && width > 0 && (act == 0 || act == 1) && (dt == X0NE_F32 || dt == X0NE_BF16),
                 "bias_act: rows %d width %d act %d dtype tag %d", n_rows, width, act, dt);
    if (n_rows == 0) return 0;
    const int64_t total = (int64_t)n_rows * width;
    if (width % 8 == 0 && ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)bias) & 15) == 0)) {
        const int threads = width / 8 >= 128 ? 128 : (width / 8 + 31) / 32 * 32;
        const dim3 vgrid((width / 8 + threads - 1) / threads, n_rows < 65535 ? n_rows : 65535);
        if (dt == X0NE_F32) x0ne_launch(bias_act_vec_kernel<float>, vgrid, dim3(threads), 0, stream, (const float*)x, bias, (float*)out, width, n_rows, act, a, b);
        else x0ne_launch(bias_act_vec_kernel<bf16>, vgrid, dim3(threads), 0, stream, (const bf16*)x, bias, (bf16*)out, width, n_rows, act, a, b);
        X0NE_LAUNCH_CHECK();
    }
    const unsigned grid = (unsigned)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
    if (dt == X0NE_F32) x0ne_launch(bias_act_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)x, bias, (float*)out, width, total, act, a, b);
    else x0ne_launch(bias_act_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)x, bias, (bf16*)out, width, total, act, a, b);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Preparation of an attention that rotates interleaved pairs and may hold several score maps per head.  src holds, per
// row, the queries at column 0 (q_heads x maps x dim), the keys at k_col (kv_heads x maps x dim) and the values at v_col
// (kv_heads x value width).  Of every (head, map) the first `rot` values are pairs (2i, 2i + 1) that turn by
// pos * freq[i]: (u, v) -> (u cos - v sin, v cos + u sin); `table` (float32 [positions][rot]: rot/2 cosines, then rot/2
// sines) replaces the computation for the positions it covers.  With unit_eps >= 0 every (head, map), after its rotation,
// is divided by sqrt(mean(x^2) + unit_eps) over its dim values.  A kv head's maps lie side by side in its key row of
// maps x dim values.  Queries go to q_out as [rows][q_heads x maps][dim], or, with `q_padded`, as [rows][q_heads x maps]
// [maps x dim] with map m's values at column m x dim and zeros beside them: such a query, met with the whole key row,
// scores against its own map alone.  One warp per (row, head and map of q or k, or value head); rows without a page
// write no keys or values.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_pairs_kv_write_kernel(const T* __restrict__ src, int ld, int k_col, int v_col, const float* __restrict__ freq,
                                           const float* __restrict__ table, int table_positions, int rot, int maps, int dim,
                                           float unit_eps, T* __restrict__ q_out, int q_heads, int q_padded, PagedCache cache,
                                           const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos, int n_rows,
                                           int write_kv) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int nq = q_heads * maps, nk = cache.kv_heads * maps;
    const int units = nq + nk + cache.kv_heads;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_rows * units) return;
    const int row = (int)(item / units), unit = (int)(item % units);
    const int pos = row_pos[row], slot = row_slot[row];
    const T* s = src + (int64_t)row * ld;
    if (unit >= nq + nk) {                        // a value head: copied as it is
        const int g = unit - nq - nk, vd = cache_v_dim(cache);
        const int64_t off = write_kv ? cache_row_offset(cache, slot, pos, g, 1) : -1;
        if (off < 0) return;
        T* dst = (T*)cache.base + off;
        for (int i = lane; i < vd; i += 32) dst[i] = s[v_col + (int64_t)g * vd + i];
        return;
    }
    const bool is_q = unit < nq;
    const int sub = is_q ? unit : unit - nq;      // head x maps + map
    const T* x = s + (is_q ? 0 : k_col) + (int64_t)sub * dim;
    T* dst;
    if (is_q) {
        const int w = q_padded ? maps * dim : dim;
        dst = q_out + ((int64_t)row * nq + sub) * w;
        if (q_padded) {
            for (int i = lane; i < w; i += 32)
                if (i / dim != sub % maps) dst[i] = from_f32<T>(0.f);
            dst += (sub % maps) * dim;
        }
    } else {
        const int64_t off = write_kv ? cache_row_offset(cache, slot, pos, sub / maps, 0) : -1;
        if (off < 0) return;
        dst = (T*)cache.base + off + (sub % maps) * dim;
    }
    const int half = rot / 2, pairs = (dim + 1) / 2;
    const bool tabled = pos >= 0 && pos < table_positions && table != nullptr;
    // two passes over the pairs this lane owns: the sum of squares of the rotated values, then the values themselves
    float scale = 1.f;
    for (int pass = unit_eps >= 0.f ? 0 : 1; pass < 2; ++pass) {
        float ss = 0.f;
        for (int p = lane; p < pairs; p += 32) {
            float u = to_f32(x[2 * p]), v = 2 * p + 1 < dim ? to_f32(x[2 * p + 1]) : 0.f;
            if (p < half) {
                float c, sn;
                if (tabled) {
                    c = table[(int64_t)pos * rot + p];
                    sn = table[(int64_t)pos * rot + half + p];
                } else {
                    sincosf((float)pos * freq[p], &sn, &c);
                }
                const float ru = u * c - v * sn, rv = v * c + u * sn;
                u = ru;
                v = rv;
            }
            if (pass == 0) {
                ss = fmaf(u, u, ss);
                ss = fmaf(v, v, ss);
            } else {
                dst[2 * p] = from_f32<T>(u * scale);
                if (2 * p + 1 < dim) dst[2 * p + 1] = from_f32<T>(v * scale);
            }
        }
        if (pass == 0) scale = 1.0f / sqrtf(warp_sum(ss) / (float)dim + unit_eps);
    }
}

X0NE_API int x0ne_rope_pairs_kv_write(const void* src, int dt, int ld, int k_col, int v_col, const float* freq, const float* table,
                                      int table_positions, int rot, int maps, int dim, float unit_eps, void* q_out, int q_heads,
                                      int q_padded, PagedCache cache, const int32_t* row_slot, const int32_t* row_pos, int n_rows,
                                      int write_kv, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && q_heads > 0 && maps > 0 && dim > 0 && rot >= 0 && rot % 2 == 0 && rot <= dim && cache.kv_heads > 0,
                 "rope_pairs: heads %d maps %d dim %d rot %d", q_heads, maps, dim, rot);
    X0NE_REQUIRE(cache.head_dim == maps * dim && cache.v_dim >= 0, "rope_pairs: the cache's key rows hold %d values, not %d maps of %d", cache.head_dim, maps, dim);
    X0NE_REQUIRE(rot == 0 || freq != nullptr, "rope_pairs: no frequencies");
    const int vd = cache_v_dim(cache);
    X0NE_REQUIRE(k_col >= q_heads * maps * dim && v_col >= k_col + cache.kv_heads * maps * dim && ld >= v_col + cache.kv_heads * vd,
                 "rope_pairs: columns %d, %d do not fit rows of %d", k_col, v_col, ld);
    if (n_rows == 0) return 0;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * (q_heads * maps + cache.kv_heads * maps + cache.kv_heads);
    X0NE_REQUIRE((items + warps - 1) / warps <= 0x7fffffff, "rope_pairs: too many rows");
    const dim3 grid((unsigned)((items + warps - 1) / warps));
    if (dt == X0NE_F32)
        x0ne_launch(rope_pairs_kv_write_kernel<float>, grid, dim3(warps * 32), 0, stream, (const float*)src, ld, k_col, v_col, freq, table,
                    table_positions, rot, maps, dim, unit_eps, (float*)q_out, q_heads, q_padded, cache, row_slot, row_pos, n_rows, write_kv);
    else if (dt == X0NE_BF16)
        x0ne_launch(rope_pairs_kv_write_kernel<bf16>, grid, dim3(warps * 32), 0, stream, (const bf16*)src, ld, k_col, v_col, freq, table,
                    table_positions, rot, maps, dim, unit_eps, (bf16*)q_out, q_heads, q_padded, cache, row_slot, row_pos, n_rows, write_kv);
    else
        X0NE_REQUIRE(false, "rope_pairs: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Differential heads.  att (float32) holds, per row, heads x 2 results of vd values (map 1, then map 2 of each head):
//   o = a1 - lambda a2;  out[row][head] = o / sqrt(mean(o^2) + eps) * post * sigmoid(gate[row][head x vd + d])
// (gate null: no gate).  One warp per (row, head); the difference, the norm and the gate are float32.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void diff_heads_kernel(const float* __restrict__ att, const T* __restrict__ gate, int64_t gate_ld, T* __restrict__ out, int n_rows,
                                  int heads, int vd, float lambda, float eps, float post) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_rows * heads) return;
    const int row = (int)(item / heads), head = (int)(item % heads);
    const float* a1 = att + ((int64_t)row * heads + head) * 2 * vd;
    const float* a2 = a1 + vd;
    float ss = 0.f;
    for (int i = lane; i < vd; i += 32) {
        const float o = a1[i] - lambda * a2[i];
        ss = fmaf(o, o, ss);
    }
    const float scale = post / sqrtf(warp_sum(ss) / (float)vd + eps);
    T* dst = out + ((int64_t)row * heads + head) * vd;
    const T* g = gate != nullptr ? gate + (int64_t)row * gate_ld + (int64_t)head * vd : nullptr;
    for (int i = lane; i < vd; i += 32) {
        float o = (a1[i] - lambda * a2[i]) * scale;
        if (g != nullptr) o *= 1.0f / (1.0f + expf(-to_f32(g[i])));
        dst[i] = from_f32<T>(o);
    }
}

X0NE_API int x0ne_diff_heads(const float* att, const void* gate, int64_t gate_ld, void* out, int dt, int n_rows, int heads, int vd,
                             float lambda, float eps, float post, cudaStream_t stream) {
    X0NE_REQUIRE(n_rows >= 0 && heads > 0 && vd > 0 && (gate == nullptr || gate_ld >= (int64_t)heads * vd), "diff_heads: rows %d heads %d of %d", n_rows, heads, vd);
    if (n_rows == 0) return 0;
    const int warps = 4;
    const int64_t items = (int64_t)n_rows * heads;
    const dim3 grid((unsigned)((items + warps - 1) / warps));
    if (dt == X0NE_F32)
        x0ne_launch(diff_heads_kernel<float>, grid, dim3(warps * 32), 0, stream, att, (const float*)gate, gate_ld, (float*)out,
                    n_rows, heads, vd, lambda, eps, post);
    else if (dt == X0NE_BF16)
        x0ne_launch(diff_heads_kernel<bf16>, grid, dim3(warps * 32), 0, stream, att, (const bf16*)gate, gate_ld, (bf16*)out,
                    n_rows, heads, vd, lambda, eps, post);
    else
        X0NE_REQUIRE(false, "diff_heads: unknown dtype tag %d", dt);
    X0NE_LAUNCH_CHECK();
}
