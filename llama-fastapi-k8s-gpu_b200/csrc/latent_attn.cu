// Latent attention of the layer-list models: every token caches ONE row [c | shared rotated key part] (c = RMS-normed
// low-rank latent) that all heads read; keys and values are linear maps of c per head. The key map is folded into the
// query (the caller multiplies each head's unrotated query by W_uk,h^T), so a score is one dot product of the folded
// query [rank + dr] with the cached row, and the softmax-weighted sum runs over the c parts; the value map is applied
// afterwards to that sum. Sliding window, and a per-head sink term in the softmax denominator (it has no value).
// Softmax, the norm of c and the rotation are 32-bit; only the cached rows may be bf16.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

#include <stdlib.h>

#include <algorithm>

namespace b2 {

namespace {
__device__ __forceinline__ void row_store(void* pool, int f32, size_t i, float v) {
    if (f32) reinterpret_cast<float*>(pool)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(pool)[i] = __float2bfloat16(v);
}
__device__ __forceinline__ float row_load(const void* pool, int f32, size_t i) {
    return f32 ? reinterpret_cast<const float*>(pool)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(pool)[i]);
}
// entry i of a vector whose first rot_dims entries are rotated in pairs (i, i + rot_dims / 2) by position `pos`
__device__ __forceinline__ float rotate_half_at(const float* v, int i, int pos, const RotaryTable& rot) {
    const int half = rot.rot_dims / 2;
    if (i >= rot.rot_dims) return v[i];
    const int p = i < half ? i : i - half;
    const float cs = rot.cos[(size_t)pos * half + p], sn = rot.sin[(size_t)pos * half + p];
    return i < half ? v[i] * cs - v[i + half] * sn : v[i] * cs + v[i - half] * sn;
}
}  // namespace

// grid (T), 128 threads
__global__ void __launch_bounds__(128) latent_store_kernel(LatentAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[4];
    const int t = blockIdx.x, pos = r.tok_pos[t];
    const int slot = r.seg_slot[r.tok_seg[t]];
    const int Dk = a.rank + a.dr;
    const float* dkv = a.proj + (size_t)t * a.ldp + a.dkv_off;
    const size_t dst = ((size_t)a.block_tables[slot][pos / a.block_tokens] * a.block_tokens + pos % a.block_tokens) * Dk;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(dkv[i], dkv[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float rinv = 1.f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)a.rank + a.eps);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) row_store(a.pool, a.cache_f32, dst + i, dkv[i] * rinv * a.c_norm_w[i]);
    for (int i = threadIdx.x; i < a.dr; i += blockDim.x) row_store(a.pool, a.cache_f32, dst + a.rank + i, rotate_half_at(dkv + a.rank, i, pos, a.rot));
    for (int j = threadIdx.x; j < a.H * a.dr; j += blockDim.x) {
        const int h = j / a.dr, i = j % a.dr;
        const float* q = a.proj + (size_t)t * a.ldp + a.q_off + (size_t)h * (a.d + a.dr) + a.d;
        a.qv[((size_t)t * a.H + h) * Dk + a.rank + i] = rotate_half_at(q, i, pos, a.rot);
    }
}
cudaError_t latent_store_launch(const LatentAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(latent_store_kernel, dim3(r.T), dim3(128), 0, s, a, r);
}

// grid (T, H, splits), 8 warps: CTA z takes the z-th range of the visible keys, warp w its keys w, w + 8, ...; a lane holds
// entries lane, lane + 32, ... of the row. The sink enters as the starting state of warp 0 of range 0: maximum = sink,
// sum = 1, no value. With several ranges the CTA leaves (max, sum, unnormalised output) for latent_merge_kernel.
constexpr int LA_WARPS = 8;
template <int E>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attn_kernel(LatentAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float sm_m[LA_WARPS], sm_l[LA_WARPS];
    extern __shared__ float sm_o[];                    // [LA_WARPS][rank]
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = r.tok_pos[t];
    const int* table = a.block_tables[r.seg_slot[r.tok_seg[t]]];
    const int Dk = a.rank + a.dr;
    const float* q = a.qv + ((size_t)t * a.H + h) * Dk;
    float qr[E], acc[E];
#pragma unroll
    for (int e = 0; e < E; e++) { const int i = lane + 32 * e; qr[e] = i < Dk ? q[i] * a.scale : 0.f; acc[e] = 0.f; }
    const int lo = max(0, pos - a.window + 1);
    const int n_splits = gridDim.z, n_all = pos - lo + 1, chunk = (n_all + n_splits - 1) / n_splits;
    const int j_begin = lo + blockIdx.z * chunk, j_end = min(pos + 1, j_begin + chunk);
    const bool has_sink = warp == 0 && blockIdx.z == 0;
    float m = has_sink ? a.sink[h] : -INFINITY, l = has_sink ? 1.f : 0.f;
    for (int j0 = j_begin + warp * 2; j0 < j_end; j0 += LA_WARPS * 2) {       // two keys per round: their loads overlap
        const int j1 = min(j0 + 1, j_end - 1);
        const size_t base0 = ((size_t)table[j0 / a.block_tokens] * a.block_tokens + j0 % a.block_tokens) * Dk;
        const size_t base1 = ((size_t)table[j1 / a.block_tokens] * a.block_tokens + j1 % a.block_tokens) * Dk;
        float k0[E], k1[E], d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int e = 0; e < E; e++) {
            const int i = lane + 32 * e;
            k0[e] = i < Dk ? row_load(a.pool, a.cache_f32, base0 + i) : 0.f;
            k1[e] = i < Dk ? row_load(a.pool, a.cache_f32, base1 + i) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < E; e++) { d0 = fmaf(qr[e], k0[e], d0); d1 = fmaf(qr[e], k1[e], d1); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { d0 += __shfl_xor_sync(0xffffffffu, d0, o); d1 += __shfl_xor_sync(0xffffffffu, d1, o); }
        const bool two = j0 + 1 < j_end;
        const float m_new = fmaxf(m, two ? fmaxf(d0, d1) : d0);
        const float corr = expf(m - m_new), p0 = expf(d0 - m_new), p1 = two ? expf(d1 - m_new) : 0.f;
        l = l * corr + p0 + p1;
#pragma unroll
        for (int e = 0; e < E; e++) acc[e] = fmaf(p1, k1[e], fmaf(p0, k0[e], acc[e] * corr));
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < E; e++) { const int i = lane + 32 * e; if (i < a.rank) sm_o[warp * a.rank + i] = acc[e]; }
    __syncthreads();
    float M = -INFINITY;
    for (int w2 = 0; w2 < LA_WARPS; w2++) M = fmaxf(M, sm_m[w2]);
    float L = 0.f;
    for (int w2 = 0; w2 < LA_WARPS; w2++) if (sm_m[w2] > -INFINITY) L += sm_l[w2] * expf(sm_m[w2] - M);
    float* part = n_splits > 1 ? a.split_scratch + (((size_t)t * a.H + h) * n_splits + blockIdx.z) * (a.rank + 2) : nullptr;
    if (part && threadIdx.x == 0) { part[0] = M; part[1] = L; }
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        float o = 0.f;
        for (int w2 = 0; w2 < LA_WARPS; w2++) if (sm_m[w2] > -INFINITY) o += sm_o[w2 * a.rank + i] * expf(sm_m[w2] - M);
        if (part) part[2 + i] = o;
        else a.o_lat[((size_t)t * a.H + h) * a.rank + i] = o / L;
    }
}

// Even row lengths: a lane holds PAIRS of neighbouring entries (one 4- or 8-byte load per key and 64 entries of the row) and a
// warp takes four keys per round, so that 4 x E2 loads are in flight per lane before the first dot product is reduced.
template <bool F32>
__device__ __forceinline__ float2 row_load2(const void* pool, size_t i) {
    if constexpr (F32) return *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(pool) + i);
    const uint32_t u = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(pool) + i);
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
constexpr int LA_KEYS = 4;
template <int E2, bool F32>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attn_pairs_kernel(LatentAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float sm_m[LA_WARPS], sm_l[LA_WARPS];
    extern __shared__ float sm_o[];                    // [LA_WARPS][rank]
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = r.tok_pos[t];
    const int* table = a.block_tables[r.seg_slot[r.tok_seg[t]]];
    const int Dk = a.rank + a.dr;
    const float* q = a.qv + ((size_t)t * a.H + h) * Dk;
    float2 qr[E2], acc[E2];
#pragma unroll
    for (int e = 0; e < E2; e++) {
        const int i = 64 * e + 2 * lane;
        qr[e] = i < Dk ? make_float2(q[i] * a.scale, q[i + 1] * a.scale) : make_float2(0.f, 0.f);
        acc[e] = make_float2(0.f, 0.f);
    }
    const int lo = max(0, pos - a.window + 1);
    const int n_splits = gridDim.z, n_all = pos - lo + 1, chunk = (n_all + n_splits - 1) / n_splits;
    const int j_begin = lo + blockIdx.z * chunk, j_end = min(pos + 1, j_begin + chunk);
    const bool has_sink = warp == 0 && blockIdx.z == 0;
    float m = has_sink ? a.sink[h] : -INFINITY, l = has_sink ? 1.f : 0.f;
    for (int j0 = j_begin + warp * LA_KEYS; j0 < j_end; j0 += LA_WARPS * LA_KEYS) {
        size_t base[LA_KEYS];
        float2 kv[LA_KEYS][E2];
        float sc[LA_KEYS];
#pragma unroll
        for (int u = 0; u < LA_KEYS; u++) {
            const int j = min(j0 + u, j_end - 1);          // past the end: the last key again, its weight is dropped below
            base[u] = ((size_t)table[j / a.block_tokens] * a.block_tokens + j % a.block_tokens) * Dk;
        }
#pragma unroll
        for (int u = 0; u < LA_KEYS; u++)
#pragma unroll
            for (int e = 0; e < E2; e++) {
                const int i = 64 * e + 2 * lane;
                kv[u][e] = i < Dk ? row_load2<F32>(a.pool, base[u] + i) : make_float2(0.f, 0.f);
            }
#pragma unroll
        for (int u = 0; u < LA_KEYS; u++) {
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < E2; e++) dot = fmaf(qr[e].x, kv[u][e].x, fmaf(qr[e].y, kv[u][e].y, dot));
            sc[u] = dot;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < LA_KEYS; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
        float m_new = m;
#pragma unroll
        for (int u = 0; u < LA_KEYS; u++) if (j0 + u < j_end) m_new = fmaxf(m_new, sc[u]);
        const float corr = expf(m - m_new);
        float p[LA_KEYS], ps = 0.f;
#pragma unroll
        for (int u = 0; u < LA_KEYS; u++) { p[u] = j0 + u < j_end ? expf(sc[u] - m_new) : 0.f; ps += p[u]; }
        l = l * corr + ps;
#pragma unroll
        for (int e = 0; e < E2; e++) {
            float ax = acc[e].x * corr, ay = acc[e].y * corr;
#pragma unroll
            for (int u = 0; u < LA_KEYS; u++) { ax = fmaf(p[u], kv[u][e].x, ax); ay = fmaf(p[u], kv[u][e].y, ay); }
            acc[e] = make_float2(ax, ay);
        }
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < E2; e++) {
        const int i = 64 * e + 2 * lane;
        if (i < a.rank) sm_o[warp * a.rank + i] = acc[e].x;
        if (i + 1 < a.rank) sm_o[warp * a.rank + i + 1] = acc[e].y;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w2 = 0; w2 < LA_WARPS; w2++) M = fmaxf(M, sm_m[w2]);
    float L = 0.f;
    for (int w2 = 0; w2 < LA_WARPS; w2++) if (sm_m[w2] > -INFINITY) L += sm_l[w2] * expf(sm_m[w2] - M);
    float* part = n_splits > 1 ? a.split_scratch + (((size_t)t * a.H + h) * n_splits + blockIdx.z) * (a.rank + 2) : nullptr;
    if (part && threadIdx.x == 0) { part[0] = M; part[1] = L; }
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        float o = 0.f;
        for (int w2 = 0; w2 < LA_WARPS; w2++) if (sm_m[w2] > -INFINITY) o += sm_o[w2 * a.rank + i] * expf(sm_m[w2] - M);
        if (part) part[2 + i] = o;
        else a.o_lat[((size_t)t * a.H + h) * a.rank + i] = o / L;
    }
}

// sum of the key ranges of one (token, head) in range order (range 0 carries the sink, so the sum is never empty)
__global__ void __launch_bounds__(128) latent_merge_kernel(LatentAttnArgs a, int n_splits) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, h = blockIdx.y, n = a.rank + 2;
    const float* part = a.split_scratch + ((size_t)t * a.H + h) * n_splits * n;
    float M = -INFINITY;
    for (int s2 = 0; s2 < n_splits; s2++) M = fmaxf(M, part[(size_t)s2 * n]);
    float L = 0.f;
    for (int s2 = 0; s2 < n_splits; s2++) { const float ms = part[(size_t)s2 * n]; if (ms > -INFINITY) L += part[(size_t)s2 * n + 1] * expf(ms - M); }
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        float o = 0.f;
        for (int s2 = 0; s2 < n_splits; s2++) { const float ms = part[(size_t)s2 * n]; if (ms > -INFINITY) o += part[(size_t)s2 * n + 2 + i] * expf(ms - M); }
        a.o_lat[((size_t)t * a.H + h) * a.rank + i] = o / L;
    }
}

// Tensor-core prompt kernel (bf16 pages, rank and rank + dr multiples of 16): a CTA takes one tile of up to 64 consecutive
// queries of a segment, one head and one chunk of LT_DV latent columns of the output (128 for latents up to 128 wide, else
// 256: every chunk recomputes the scores, so wide chunks pay back their registers); 4 warps x 16 query rows; cached rows in
// blocks of 64, staged in shared memory once for all 64 queries. S = Q K^T over the whole row, O += P K[:, chunk], with
// mma.sync m16n8k16 (bf16 in, f32 accumulate); mask, running maximum, exponentials and sums are 32-bit; the running state
// starts at (maximum = sink, sum = 1).
constexpr int LT_Q = 64, LT_K = 64;
namespace {
__device__ __forceinline__ void cp_async_16z(void* smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
}  // namespace

template <int LT_DV>
__global__ void __launch_bounds__(128) latent_attn_mma_kernel(LatentAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char lt_smem[];
    const int Dk = a.rank + a.dr, LD = Dk + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lt_smem);     // [64][LD] scaled queries
    __nv_bfloat16* Ks = Qs + LT_Q * LD;                                 // [64][LD] cached rows
    const int tile = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * LT_DV, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_cols = min(LT_DV, a.rank - c0);
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(LT_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int* table = a.block_tables[r.seg_slot[seg]];
    const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(a.pool);
    for (int i = threadIdx.x; i < LT_Q * (Dk / 2); i += blockDim.x) {
        const int rr = i / (Dk / 2), c = (i % (Dk / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (rr < nq) {
            const float* q = a.qv + ((size_t)(row0 + rr) * a.H + h) * Dk + c;
            v = make_float2(q[0] * a.scale, q[1] * a.scale);
        }
        *reinterpret_cast<__nv_bfloat162*>(Qs + rr * LD + c) = __floats2bfloat162_rn(v.x, v.y);
    }
    const int b0 = max(0, p0 - a.window + 1) / LT_K, b1 = p_last / LT_K;
    float o[LT_DV / 8][4];
#pragma unroll
    for (int i = 0; i < LT_DV / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const float sink = a.sink[h];
    float m_run[2] = {sink, sink}, l_run[2] = {0.f, 0.f};      // the sink's own 1 joins the sum after the lane reduction
    const int gq = lane >> 2, tq = lane & 3;
    const int qrow[2] = {warp * 16 + gq, warp * 16 + gq + 8};
    for (int kb = b0; kb <= b1; kb++) {
        const int j0 = kb * LT_K;
        __syncthreads();                      // everybody is done with the previous block's rows (and Q is written)
        for (int i = threadIdx.x; i < LT_K * (Dk / 8); i += blockDim.x) {
            const int rr = i / (Dk / 8), c = (i % (Dk / 8)) * 8;
            const int j = j0 + rr, jj = min(j, p_last);
            const size_t base = ((size_t)table[jj / a.block_tokens] * a.block_tokens + jj % a.block_tokens) * Dk + c;
            cp_async_16z(Ks + rr * LD + c, pool + base, j <= p_last ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        float sacc[LT_K / 8][4];
#pragma unroll
        for (int ni = 0; ni < LT_K / 8; ni++) sacc[ni][0] = sacc[ni][1] = sacc[ni][2] = sacc[ni][3] = 0.f;
#pragma unroll 2
        for (int ks = 0; ks < Dk; ks += 16) {
            uint32_t af[4];
            ldsm_x4(af, Qs + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
#pragma unroll
            for (int nj = 0; nj < LT_K / 16; nj++) {
                uint32_t bf[4];
                ldsm_x4(bf, Ks + (nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks + ((lane >> 3) & 1) * 8);
                mma_16816(sacc[2 * nj], af, bf[0], bf[1]);
                mma_16816(sacc[2 * nj + 1], af, bf[2], bf[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int ni = 0; ni < LT_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int rr = qrow[e >> 1], i = p0 + rr, j = j0 + ni * 8 + 2 * tq + (e & 1);
                const bool vis = rr < nq && j <= i && i - j < a.window;
                const float v = vis ? sacc[ni][e] : -INFINITY;
                sacc[ni][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float corr[2];
#pragma unroll
        for (int q2 = 0; q2 < 2; q2++) {
            mx[q2] = fmaxf(mx[q2], __shfl_xor_sync(0xffffffffu, mx[q2], 1));
            mx[q2] = fmaxf(mx[q2], __shfl_xor_sync(0xffffffffu, mx[q2], 2));
            const float m_new = fmaxf(m_run[q2], mx[q2]);       // finite: the sink is
            corr[q2] = expf(m_run[q2] - m_new);
            m_run[q2] = m_new;
            l_run[q2] *= corr[q2];
        }
#pragma unroll
        for (int ni = 0; ni < LT_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float pv = expf(sacc[ni][e] - m_run[e >> 1]);
                sacc[ni][e] = pv;
                l_run[e >> 1] += pv;
            }
#pragma unroll
        for (int i = 0; i < LT_DV / 8; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
        for (int kc = 0; kc < LT_K / 16; kc++) {
            uint32_t pf[4];
            pf[0] = pack_bf16(sacc[2 * kc][0], sacc[2 * kc][1]);
            pf[1] = pack_bf16(sacc[2 * kc][2], sacc[2 * kc][3]);
            pf[2] = pack_bf16(sacc[2 * kc + 1][0], sacc[2 * kc + 1][1]);
            pf[3] = pack_bf16(sacc[2 * kc + 1][2], sacc[2 * kc + 1][3]);
#pragma unroll
            for (int nd = 0; nd < LT_DV / 16; nd++) {
                if (nd * 16 < n_cols) {
                    uint32_t vf[4];
                    ldsm_x4_t(vf, Ks + (kc * 16 + (lane & 15)) * LD + c0 + nd * 16 + (lane >> 4) * 8);
                    mma_16816(o[2 * nd], pf, vf[0], vf[1]);
                    mma_16816(o[2 * nd + 1], pf, vf[2], vf[3]);
                }
            }
        }
    }
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        l_run[q2] += __shfl_xor_sync(0xffffffffu, l_run[q2], 1);
        l_run[q2] += __shfl_xor_sync(0xffffffffu, l_run[q2], 2);
        l_run[q2] += expf(sink - m_run[q2]);
    }
#pragma unroll
    for (int i = 0; i < LT_DV / 8; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int rr = qrow[e >> 1], c = i * 8 + 2 * tq + (e & 1);
            if (rr < nq && c < n_cols) a.o_lat[((size_t)(row0 + rr) * a.H + h) * a.rank + c0 + c] = o[i][e] / l_run[e >> 1];
        }
}

cudaError_t latent_attn_launch(const LatentAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    const int Dk = a.rank + a.dr;
    if (Dk > 640) return cudaErrorInvalidValue;
    static const bool no_mma = getenv("B2_NO_ATTN_MMA") != nullptr;        // tuning aid: scalar attention for prompts too
    if (!no_mma && !a.cache_f32 && r.T > 8 && a.rank % 16 == 0 && Dk % 16 == 0) {
        static bool attr_done = false;
        if (!attr_done) {
            cudaFuncSetAttribute(latent_attn_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 64 * (640 + 8) * 2);
            cudaFuncSetAttribute(latent_attn_mma_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 64 * (640 + 8) * 2);
            attr_done = true;
        }
        const size_t smem = (size_t)2 * 64 * (Dk + 8) * 2;
        if (a.rank <= 128) return launch_chain(latent_attn_mma_kernel<128>, dim3(r.n_tiles, a.H, 1), dim3(128), smem, s, a, r);
        return launch_chain(latent_attn_mma_kernel<256>, dim3(r.n_tiles, a.H, (a.rank + 255) / 256), dim3(128), smem, s, a, r);
    }
    // a step of a few tokens does not fill the GPU with one CTA per (token, head): split the keys (up to 16 ranges)
    int splits = 1;
    if (a.split_scratch && r.T * a.H < 148) {
        splits = std::min({16, (2 * 148) / (r.T * a.H), std::max(1, a.window / 32)});
        while (splits > 1 && (size_t)r.T * a.H * splits * (a.rank + 2) > (size_t)a.split_capacity) splits--;
    }
    const dim3 grid(r.T, a.H, splits), block(LA_WARPS * 32);
    const size_t smem = (size_t)LA_WARPS * a.rank * 4;
    cudaError_t ce;
    if (Dk % 2 == 0) {
        if (Dk <= 192) ce = a.cache_f32 ? launch_chain(latent_attn_pairs_kernel<3, true>, grid, block, smem, s, a, r)
                                        : launch_chain(latent_attn_pairs_kernel<3, false>, grid, block, smem, s, a, r);
        else if (Dk <= 384) ce = a.cache_f32 ? launch_chain(latent_attn_pairs_kernel<6, true>, grid, block, smem, s, a, r)
                                             : launch_chain(latent_attn_pairs_kernel<6, false>, grid, block, smem, s, a, r);
        else ce = a.cache_f32 ? launch_chain(latent_attn_pairs_kernel<10, true>, grid, block, smem, s, a, r)
                              : launch_chain(latent_attn_pairs_kernel<10, false>, grid, block, smem, s, a, r);
    } else if (Dk <= 160) ce = launch_chain(latent_attn_kernel<5>, grid, block, smem, s, a, r);
    else if (Dk <= 320) ce = launch_chain(latent_attn_kernel<10>, grid, block, smem, s, a, r);
    else ce = launch_chain(latent_attn_kernel<20>, grid, block, smem, s, a, r);
    if (ce != cudaSuccess || splits == 1) return ce;
    return launch_chain(latent_merge_kernel, dim3(r.T, a.H), dim3(128), 0, s, a, splits);
}

}  // namespace b2
