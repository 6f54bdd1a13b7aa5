// Latent attention of the layer-list models: every token caches ONE row [c | shared rotated key part] (c = RMS-normed
// low-rank latent) that all heads read; keys and values are linear maps of c per head. The key map is folded into the
// query (the caller multiplies each head's unrotated query by W_uk,h^T), so a score is one dot product of the folded
// query [rank + dr] with the cached row, and the softmax-weighted sum runs over the c parts; the value map is applied
// afterwards to that sum. Sliding window, and a per-head sink term in the softmax denominator (it has no value).
// Softmax, the norm of c and the rotation are 32-bit; only the cached rows may be bf16.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

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

// grid (T, H), 8 warps: warp w takes visible keys w, w + 8, ...; a lane holds entries lane, lane + 32, ... of the row.
// The sink enters as warp 0's starting state: maximum = sink, sum = 1, no value.
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
    float m = warp == 0 ? a.sink[h] : -INFINITY, l = warp == 0 ? 1.f : 0.f;
    for (int j = lo + warp; j <= pos; j += LA_WARPS) {
        const size_t base = ((size_t)table[j / a.block_tokens] * a.block_tokens + j % a.block_tokens) * Dk;
        float kv[E], dot = 0.f;
#pragma unroll
        for (int e = 0; e < E; e++) {
            const int i = lane + 32 * e;
            kv[e] = i < Dk ? row_load(a.pool, a.cache_f32, base + i) : 0.f;
            dot = fmaf(qr[e], kv[e], dot);
        }
        const float sc = warp_sum(dot);
        const float m_new = fmaxf(m, sc);
        const float corr = expf(m - m_new), p = expf(sc - m_new);
        l = l * corr + p;
#pragma unroll
        for (int e = 0; e < E; e++) acc[e] = fmaf(p, kv[e], acc[e] * corr);
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
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        float o = 0.f;
        for (int w2 = 0; w2 < LA_WARPS; w2++) if (sm_m[w2] > -INFINITY) o += sm_o[w2 * a.rank + i] * expf(sm_m[w2] - M);
        a.o_lat[((size_t)t * a.H + h) * a.rank + i] = o / L;
    }
}

cudaError_t latent_attn_launch(const LatentAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    const int Dk = a.rank + a.dr;
    if (Dk > 640) return cudaErrorInvalidValue;
    const dim3 grid(r.T, a.H), block(LA_WARPS * 32);
    const size_t smem = (size_t)LA_WARPS * a.rank * 4;
    if (Dk <= 160) return launch_chain(latent_attn_kernel<5>, grid, block, smem, s, a, r);
    if (Dk <= 320) return launch_chain(latent_attn_kernel<10>, grid, block, smem, s, a, r);
    return launch_chain(latent_attn_kernel<20>, grid, block, smem, s, a, r);
}

}  // namespace b2
