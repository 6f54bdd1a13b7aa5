// Recurrent token mixers of the layer-list models that keep a MATRIX per head: the gated delta rule (rows of the memory
// decay each at their own input-dependent rate; the write is the part of the value the memory does not return yet) and
// the Mamba-2 state-space recurrence (one scalar decay per head, input and output maps shared by the heads of a group).
// Both run through one kernel (col_state_kernel). Also here: the short causal convolution in front of them, their
// 32-bit input preparation (unit norms, softplus, exponentials, sigmoid) and the gated group norm behind them.
// State, decays, step sizes and norms are 32-bit; a segment's tokens are walked in order from the state its slot holds,
// so a sequence cut into portions gives the same numbers as the whole.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

#include <algorithm>

namespace b2 {

namespace {
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 0.f ? z + log1pf(expf(-z)) : log1pf(expf(z)); }
__device__ __forceinline__ void cp_async_4(float* smem_dst, const float* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
}  // namespace

// ---------------------------------------------------------------- short causal convolution
// grid (T, ceil(C / 256)): a thread per (token, channel)
__global__ void __launch_bounds__(256) causal_conv_kernel(ConvArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= a.C) return;
    const int seg = r.tok_seg[t], slot = r.seg_slot[seg], i = t - r.seg_start[seg];
    const int hist = a.taps - 1;
    float acc = a.bias ? a.bias[c] : 0.f;
    for (int j = 0; j < a.taps; j++) {
        const int srci = i - hist + j;
        const float v = srci >= 0 ? a.in[(size_t)(t - i + srci) * a.ld_in + c]
                                  : a.state[((size_t)slot * hist + (hist + srci)) * a.C + c];
        acc = fmaf(a.w[(size_t)c * a.taps + j], v, acc);
    }
    a.out[(size_t)t * a.ld_out + c] = silu_f(acc);
}
cudaError_t causal_conv_launch(const ConvArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(causal_conv_kernel, dim3(r.T, (a.C + 255) / 256), dim3(256), 0, s, a, r);
}
// grid (n_seg, ceil(C / 256)); entry k of the new state is read at k + len > k of the old one before it is written
__global__ void __launch_bounds__(256) causal_conv_advance_kernel(ConvArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int seg = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= a.C) return;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int hist = a.taps - 1;
    float* st = a.state + (size_t)slot * hist * a.C + c;
    for (int k = 0; k < hist; k++) {
        const int srci = len + k - hist;
        st[(size_t)k * a.C] = srci >= 0 ? a.in[(size_t)(start + srci) * a.ld_in + c] : st[(size_t)(k + len) * a.C];
    }
}
cudaError_t causal_conv_advance_launch(const ConvArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.taps <= 1) return cudaSuccess;
    return launch_chain(causal_conv_advance_kernel, dim3(r.n_seg, (a.C + 255) / 256), dim3(256), 0, s, a, r);
}

// ---------------------------------------------------------------- inputs of the recurrences
// grid (T): unit vectors, decays, write strengths
__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaPrepArgs a) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const float qmul = 1.f / sqrtf((float)a.d);
    for (int hv = warp; hv < 2 * a.G; hv += nw) {          // a warp per (q | k, head)
        const bool is_q = hv < a.G;
        float* v = (is_q ? a.q : a.k) + (size_t)t * a.ld_qk + (size_t)(is_q ? hv : hv - a.G) * a.d;
        float ss = 0.f;
        for (int i = lane; i < a.d; i += 32) ss = fmaf(v[i], v[i], ss);
        const float rinv = (is_q ? qmul : 1.f) / sqrtf(warp_sum(ss) + a.unit_eps);
        for (int i = lane; i < a.d; i += 32) v[i] *= rinv;
    }
    for (int i = threadIdx.x; i < a.H * a.d; i += blockDim.x) {
        float* p = a.a + (size_t)t * a.ld_a + i;
        *p = expf(-expf(a.A_log[i / a.d]) * softplus_f(*p + a.dt_bias[i]));
    }
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        float* p = a.beta + (size_t)t * a.ld_b + h;
        *p = sigmoid_f(*p);
    }
}
cudaError_t delta_prepare_launch(const DeltaPrepArgs& a, int T, cudaStream_t s) {
    return launch_chain(delta_prepare_kernel, dim3(T), dim3(256), 0, s, a);
}

__global__ void ssd_prepare_kernel(float* dt, int ld_dt, const float* dt_bias, const float* A_log, int H, float* decay, int T) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * H) return;
    const int t = i / H, h = i % H;
    const float v = softplus_f(dt[(size_t)t * ld_dt + h] + dt_bias[h]);
    dt[(size_t)t * ld_dt + h] = v;
    decay[i] = expf(-expf(A_log[h]) * v);
}
cudaError_t ssd_prepare_launch(float* dt, int ld_dt, const float* dt_bias, const float* A_log, int H, float* decay, int T, cudaStream_t s) {
    return launch_chain(ssd_prepare_kernel, dim3((T * H + 127) / 128), dim3(128), 0, s, dt, ld_dt, dt_bias, A_log, H, decay, T);
}

// ---------------------------------------------------------------- the recurrence
// grid (n_seg, H, ceil(P / CS_COLS)), 256 threads: thread (column, row lane) keeps NCH chunks of four rows of its column in
// registers (chunk index = row lane + 8 i, so the 8 row lanes of a column read 32 neighbouring floats); the two sums over
// the rows -- what the memory returns for the write key, and the read-out -- are shuffle reductions over the 8 row lanes.
// The per-token row vectors (write key, read key, row decays) are the same for every column of the head: they come into
// shared memory as asynchronous copies, CS_TB tokens at a time, the next block while this one is computed.
constexpr int CS_LANES = 8, CS_COLS = 32, CS_TB = 8;
template <int NCH>
__global__ void __launch_bounds__(CS_LANES * CS_COLS) col_state_kernel(ColStateArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) float cs_sm[];
    const int R = a.R, P = a.P, Rp = (R + 3) / 4 * 4, n_chunks = Rp / 4;
    const bool has_rd = a.row_decay != nullptr;
    float* wks = cs_sm;                              // [2][CS_TB][Rp]
    float* rks = wks + 2 * CS_TB * Rp;               // [2][CS_TB][Rp]
    float* rds = rks + 2 * CS_TB * Rp;               // [2][CS_TB][Rp] (only with row decays)
    float* vs = rds + (has_rd ? 2 * CS_TB * Rp : 0); // [2][CS_TB][CS_COLS]
    float* sc = vs + 2 * CS_TB * CS_COLS;            // [2][CS_TB][2]: value scale, head decay
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CS_COLS;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int rl = threadIdx.x % CS_LANES, lc = threadIdx.x / CS_LANES, col = c0 + lc;
    const bool col_ok = col < P;
    const int g = h / (a.H / a.G);
    float* Sg = a.state + (((size_t)slot * a.H + h) * P + (col_ok ? col : 0)) * Rp;
    float4 S[NCH];
#pragma unroll
    for (int i = 0; i < NCH; i++) {
        const int ch = rl + CS_LANES * i;
        S[i] = (col_ok && ch < n_chunks) ? *reinterpret_cast<const float4*>(Sg + 4 * ch) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int j = threadIdx.x; j < (has_rd ? 6 : 4) * CS_TB * Rp + 2 * CS_TB * (CS_COLS + 2); j += blockDim.x) cs_sm[j] = 0.f;
    __syncthreads();
    auto stage = [&](int i0, int buf) {
        const int nb = min(CS_TB, len - i0);
        for (int j = threadIdx.x; j < nb * R; j += blockDim.x) {
            const int u = j / R, e = j % R;
            const size_t t = start + i0 + u;
            const int d = (buf * CS_TB + u) * Rp + e;
            cp_async_4(wks + d, a.wk + t * a.ld_wk + (size_t)g * R + e);
            cp_async_4(rks + d, a.rk + t * a.ld_rk + (size_t)g * R + e);
            if (has_rd) cp_async_4(rds + d, a.row_decay + t * a.ld_rd + (size_t)h * R + e);
        }
        for (int j = threadIdx.x; j < nb * CS_COLS; j += blockDim.x) {
            const int u = j / CS_COLS, e = j % CS_COLS;
            const size_t t = start + i0 + u;
            if (c0 + e < P) cp_async_4(vs + (buf * CS_TB + u) * CS_COLS + e, a.val + t * a.ld_v + (size_t)h * P + c0 + e);
            if (e == 0) cp_async_4(sc + (buf * CS_TB + u) * 2, a.val_scale + t * a.ld_vs + h);
            if (e == 1 && a.head_decay) cp_async_4(sc + (buf * CS_TB + u) * 2 + 1, a.head_decay + t * a.ld_hd + h);
        }
    };
    const float skip = a.skip ? a.skip[h] : 0.f;
    if (len > 0) stage(0, 0);
    cp_async_commit();
    for (int i0 = 0; i0 < len; i0 += CS_TB) {
        const int nb = min(CS_TB, len - i0), buf = (i0 / CS_TB) & 1;
        cp_async_wait_all();
        __syncthreads();                 // this block's inputs have landed; everybody is done with the other buffer
        if (i0 + CS_TB < len) stage(i0 + CS_TB, buf ^ 1);
        cp_async_commit();
        for (int u = 0; u < nb; u++) {
            const int bu = buf * CS_TB + u;
            const float4* wk4 = reinterpret_cast<const float4*>(wks + bu * Rp);
            const float4* rk4 = reinterpret_cast<const float4*>(rks + bu * Rp);
            const float4* rd4 = reinterpret_cast<const float4*>(rds + bu * Rp);
            const float v = vs[bu * CS_COLS + lc], vscale = sc[bu * 2];
            const float hd = a.head_decay ? sc[bu * 2 + 1] : 1.f;
            float4 kw[NCH];
            float pred = 0.f;
#pragma unroll
            for (int i = 0; i < NCH; i++) {
                const int ch = rl + CS_LANES * i;
                if (ch < n_chunks) {
                    kw[i] = wk4[ch];
                    float4 dc = make_float4(hd, hd, hd, hd);
                    if (has_rd) { const float4 q = rd4[ch]; dc = make_float4(q.x * hd, q.y * hd, q.z * hd, q.w * hd); }
                    S[i].x *= dc.x; S[i].y *= dc.y; S[i].z *= dc.z; S[i].w *= dc.w;
                    pred = fmaf(S[i].x, kw[i].x, fmaf(S[i].y, kw[i].y, fmaf(S[i].z, kw[i].z, fmaf(S[i].w, kw[i].w, pred))));
                } else kw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float uval = vscale * v;
            if (a.delta) {
#pragma unroll
                for (int o = CS_LANES / 2; o > 0; o >>= 1) pred += __shfl_xor_sync(0xffffffffu, pred, o);
                uval = vscale * (v - pred);
            }
            float out = 0.f;
#pragma unroll
            for (int i = 0; i < NCH; i++) {
                const int ch = rl + CS_LANES * i;
                if (ch < n_chunks) {
                    const float4 q = rk4[ch];
                    S[i].x = fmaf(kw[i].x, uval, S[i].x); S[i].y = fmaf(kw[i].y, uval, S[i].y);
                    S[i].z = fmaf(kw[i].z, uval, S[i].z); S[i].w = fmaf(kw[i].w, uval, S[i].w);
                    out = fmaf(S[i].x, q.x, fmaf(S[i].y, q.y, fmaf(S[i].z, q.z, fmaf(S[i].w, q.w, out))));
                }
            }
#pragma unroll
            for (int o = CS_LANES / 2; o > 0; o >>= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
            if (rl == 0 && col_ok) a.y[(size_t)(start + i0 + u) * a.ld_y + (size_t)h * P + col] = fmaf(skip, v, out);
        }
    }
#pragma unroll
    for (int i = 0; i < NCH; i++) {
        const int ch = rl + CS_LANES * i;
        if (col_ok && ch < n_chunks) *reinterpret_cast<float4*>(Sg + 4 * ch) = S[i];
    }
}

cudaError_t col_state_launch(const ColStateArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.R <= 0 || a.R > 256 || a.P <= 0 || a.H <= 0 || a.G <= 0 || a.H % a.G) return cudaErrorInvalidValue;
    const int Rp = (a.R + 3) / 4 * 4, n_chunks = Rp / 4;
    const size_t smem = (size_t)((a.row_decay ? 6 : 4) * CS_TB * Rp + 2 * CS_TB * (CS_COLS + 2)) * 4;
    const dim3 grid(r.n_seg, a.H, (a.P + CS_COLS - 1) / CS_COLS), block(CS_LANES * CS_COLS);
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(col_state_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        attr_done = true;
    }
    if (n_chunks <= 8) return launch_chain(col_state_kernel<1>, grid, block, smem, s, a, r);
    if (n_chunks <= 16) return launch_chain(col_state_kernel<2>, grid, block, smem, s, a, r);
    if (n_chunks <= 32) return launch_chain(col_state_kernel<4>, grid, block, smem, s, a, r);
    return launch_chain(col_state_kernel<8>, grid, block, smem, s, a, r);
}

// ---------------------------------------------------------------- gated group norm
// grid (T, groups)
__global__ void __launch_bounds__(128) group_norm_gate_kernel(GroupNormArgs a) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[4];
    const int t = blockIdx.x, g = blockIdx.y, n = a.n;
    const float* x = a.x + (size_t)t * a.ld_x + (size_t)g * n;
    const float* gate = a.gate + (size_t)t * a.ld_g + (size_t)g * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = a.gate_first ? x[i] * silu_f(gate[i]) : x[i];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float rinv = 1.f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)n + a.eps);
    const float* w = a.w + (size_t)g * a.w_gstride;
    float* y = a.y + (size_t)t * a.ld_y + (size_t)g * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        y[i] = a.gate_first ? x[i] * silu_f(gate[i]) * rinv * w[i] : x[i] * rinv * w[i] * sigmoid_f(gate[i]);
}
cudaError_t group_norm_gate_launch(const GroupNormArgs& a, int T, cudaStream_t s) {
    return launch_chain(group_norm_gate_kernel, dim3(T, a.groups), dim3(128), 0, s, a);
}

}  // namespace b2
