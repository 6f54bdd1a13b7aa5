// Layer-list models (include/b200_gguf.h: b2_engine_create_layered, b2_step): the graph of a decoder given as a list of
// layers -- window attention beside a selective scan, or an mLSTM matrix memory, each optionally followed by a squared-ReLU
// feed-forward block, with the layer norm AFTER each residual sum -- over dense bf16 / f32 tensors, stepped over ragged
// batches. Shares the engine object with the llama graph (engine.cu): tensors, sequence slots and their page tables,
// sampler state, stream, error reporting. Owns: fused projection matrices, per-layer cache pages, per-slot recurrent
// state, the step workspace.
#include "engine_state.h"
#include "layered.h"
#include "ptx.cuh"
#include "quant_blocks.cuh"

#include <math.h>
#include <string.h>

#include <algorithm>

namespace b2 {

struct DenseW { const void* w = nullptr; int type = 0, N = 0, K = 0; };

struct LyLayer {
    b2_layer_desc d = {};
    float *norm1 = nullptr, *norm2 = nullptr;
    // window attention + selective scan
    DenseW in_proj, attn_o, scan_x, scan_dt, scan_o;      // in_proj rows: q | k | x | z
    int q_off = 0, k_off = 0, x_off = 0, z_off = 0;
    float *q_norm = nullptr, *k_norm = nullptr, *left_w = nullptr, *right_w = nullptr;
    float *rot_cos = nullptr, *rot_sin = nullptr;
    float *conv_w = nullptr, *conv_b = nullptr, *dt_b = nullptr, *A_log = nullptr, *Dskip = nullptr;
    void *k_pool = nullptr, *v_pool = nullptr;
    float *conv_state = nullptr, *ssm_state = nullptr;
    // matrix memory
    DenseW mm_proj, mm_o;                                  // mm_proj rows: q | k | v | g | i | f
    int mq = 0, mk = 0, mv = 0, mg = 0, mi = 0, mf = 0;
    float *i_b = nullptr, *f_b = nullptr, *mm_norm = nullptr;
    float *S = nullptr, *nvec = nullptr, *mmax = nullptr;
    // feed-forward
    DenseW up, down;
    float *up_b = nullptr, *down_b = nullptr;
};

struct StepGraph { cudaGraphExec_t exec = nullptr; int n_launch = 0; bool failed = false; };

struct LayeredModel {
    b2_layered_config c = {};
    std::vector<LyLayer> layers;
    std::vector<void*> owned;          // device allocations freed at destroy
    DenseW embed, head;
    float* final_norm = nullptr;
    bool exact = false;                // B2_FLAG_F32
    int** block_tables = nullptr;      // device [max_seqs] -> page table
    // step workspace (max_step_tokens rows)
    float *x = nullptr, *proj = nullptr, *buf[4] = {}, *oL = nullptr, *oR = nullptr, *ff = nullptr, *rows = nullptr, *logits = nullptr;
    __nv_bfloat16* xb = nullptr;       // a product's input rounded to bf16 [max_step_tokens][widest input]
    std::unordered_map<std::string, StepGraph> graphs;     // replayable small steps, by shape (b2_step)
    bool graphs_on = true;
    float* attn_split = nullptr;       // few-token steps: partial attention results per key range
    int attn_split_floats = 0;
    int* meta = nullptr;               // device ints: ragged description + wanted rows
    int* meta_host = nullptr;          // pinned
    float* logits_host = nullptr;      // pinned [LOGIT_ROWS][n_vocab]
    float* trace = nullptr;            // [n_layer][max_step_tokens][n_embd] when tracing
    int last_T = 0;
    bool profile = false;
    std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> prof_ev;
    float prof_ms[8] = {};
    int prof_n[8] = {};
};

constexpr int LOGIT_ROWS = 256;

__global__ void to_f32_kernel(int type, const void* src, long n, float* dst) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= n) return;
    dst[i] = type == T_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i])
           : type == T_F16 ? __half2float(reinterpret_cast<const __half*>(src)[i])
                           : reinterpret_cast<const float*>(src)[i];
}

static int dev_alloc(LayeredModel* m, void** p, size_t bytes, bool zero = false) {
    CK(cudaMalloc(p, bytes ? bytes : 16));
    m->owned.push_back(*p);
    if (zero) CK(cudaMemset(*p, 0, bytes ? bytes : 16));
    return B2_OK;
}

static int find(b2_engine* e, const std::string& name, int64_t ne0, int64_t ne1, DevTensor& out) {
    auto it = e->tensors.find(name);
    if (it == e->tensors.end()) return b2_fail(B2_ERR_STATE, "missing tensor " + name);
    const DevTensor& t = it->second;
    if (t.ne0 != ne0 || t.ne1 != ne1)
        return b2_fail(B2_ERR_ARG, "tensor " + name + " has shape [" + std::to_string(t.ne1) + "," + std::to_string(t.ne0) +
                                       "], expected [" + std::to_string(ne1) + "," + std::to_string(ne0) + "]");
    if (t.type != T_BF16 && t.type != T_F32) return b2_fail(B2_ERR_UNSUPPORTED, "tensor " + name + " must be BF16 or F32");
    out = t;
    return B2_OK;
}

// a vector (or small table) as f32 on the device, whatever the file holds
static int vec_f32(b2_engine* e, LayeredModel* m, const std::string& name, int64_t n0, int64_t n1, float** out) {
    DevTensor t;
    int rc = find(e, name, n0, n1, t); if (rc) return rc;
    const long n = (long)(n0 * n1);
    if ((rc = dev_alloc(m, (void**)out, (size_t)n * 4))) return rc;
    to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(t.type, t.ptr, n, *out);
    CK(cudaGetLastError());
    return B2_OK;
}

static int matrix(b2_engine* e, const std::string& name, int N, int K, DenseW& out) {
    DevTensor t;
    int rc = find(e, name, K, N, t); if (rc) return rc;
    out.w = t.ptr; out.type = t.type; out.N = N; out.K = K;
    return B2_OK;
}

// several matrices over the same input stacked into one [sum N][K] matrix: one product instead of several
static int fuse(b2_engine* e, LayeredModel* m, const std::vector<std::pair<std::string, int>>& parts, int K, DenseW& out,
                std::vector<int>& offs) {
    int total = 0, type = -1;
    std::vector<DevTensor> ts(parts.size());
    for (size_t i = 0; i < parts.size(); i++) {
        int rc = find(e, parts[i].first, K, parts[i].second, ts[i]); if (rc) return rc;
        if (type < 0) type = ts[i].type;
        if (ts[i].type != type) return b2_fail(B2_ERR_UNSUPPORTED, "tensor " + parts[i].first + ": projections of one input must share a dtype");
        offs.push_back(total);
        total += parts[i].second;
    }
    const size_t esz = type == T_BF16 ? 2 : 4;
    void* p = nullptr;
    int rc = dev_alloc(m, &p, (size_t)total * K * esz + 64); if (rc) return rc;
    for (size_t i = 0; i < parts.size(); i++)
        CK(cudaMemcpyAsync((char*)p + (size_t)offs[i] * K * esz, ts[i].ptr, (size_t)parts[i].second * K * esz, cudaMemcpyDeviceToDevice, e->stream));
    out.w = p; out.type = type; out.N = total; out.K = K;
    return B2_OK;
}

// blended rotary frequencies (interpolated below the slow boundary, original above the fast one, linear ramp between)
// and the magnitude factor; cos / sin per position in double precision
static int build_rotary(b2_engine* e, LayeredModel* m, LyLayer& L) {
    const b2_layer_desc& d = L.d;
    const int half = d.rot_dims / 2;
    if (half <= 0) return B2_OK;
    std::vector<double> f(half);
    double mag = 1.0;
    for (int i = 0; i < half; i++) f[i] = pow((double)d.rope_base, -2.0 * i / (double)d.rot_dims);
    if (d.rope_factor > 0.0) {
        auto corr = [&](double turns) { return d.rot_dims * log((double)d.rope_orig_ctx / (2.0 * M_PI * turns)) / (2.0 * log((double)d.rope_base)); };
        const double lo = std::max(floor(corr(d.rope_fast)), 0.0), hi = std::min(ceil(corr(d.rope_slow)), (double)d.rot_dims - 1.0);
        for (int i = 0; i < half; i++) {
            double ramp = (i - lo) / std::max(hi - lo, 0.001);
            ramp = std::min(1.0, std::max(0.0, ramp));
            f[i] = f[i] / d.rope_factor * ramp + f[i] * (1.0 - ramp);
        }
        mag = 0.1 * log((double)d.rope_factor) + 1.0;
    }
    const int n_ctx = m->c.n_ctx;
    std::vector<float> cs((size_t)n_ctx * half), sn((size_t)n_ctx * half);
    for (int p = 0; p < n_ctx; p++)
        for (int i = 0; i < half; i++) {
            const double a = (double)p * f[i];
            cs[(size_t)p * half + i] = (float)(cos(a) * mag);
            sn[(size_t)p * half + i] = (float)(sin(a) * mag);
        }
    int rc;
    if ((rc = dev_alloc(m, (void**)&L.rot_cos, cs.size() * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&L.rot_sin, sn.size() * 4))) return rc;
    CK(cudaMemcpy(L.rot_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.rot_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
    return B2_OK;
}

int layered_finalize(b2_engine* e) {
    LayeredModel* m = e->layered;
    const b2_layered_config& c = m->c;
    const int W = c.n_embd, V = c.n_vocab, S = c.max_seqs, Tm = c.max_step_tokens;
    CK(cudaSetDevice(c.device));
    int rc;
    if ((rc = matrix(e, "embed", V, W, m->embed))) return rc;
    if ((rc = matrix(e, "head", V, W, m->head))) return rc;
    if ((rc = vec_f32(e, m, "final.norm", W, 1, &m->final_norm))) return rc;
    const size_t cache_esz = m->exact ? 4 : 2;
    size_t max_proj = 1, max_buf = 1, max_ff = 1, max_attn = 0, max_attn_d = 0;
    for (int li = 0; li < c.n_layer; li++) {
        LyLayer& L = m->layers[li];
        const b2_layer_desc& d = L.d;
        const std::string p = "l" + std::to_string(li) + ".";
        if ((rc = vec_f32(e, m, p + "norm1", W, 1, &L.norm1))) return rc;
        if (d.mixer == B2_MIX_WINDOW_SCAN) {
            const std::string a = p + "mix.left.", b = p + "mix.right.";
            const int qd = d.n_head * d.head_dim, kd = d.n_head_kv * d.head_dim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", qd}, {a + "k", kd}, {b + "in", 2 * d.d_inner}}, W, L.in_proj, offs))) return rc;
            L.q_off = offs[0]; L.k_off = offs[1]; L.x_off = offs[2]; L.z_off = offs[2] + d.d_inner;
            if ((rc = vec_f32(e, m, a + "q.norm", d.head_dim, 1, &L.q_norm))) return rc;
            if ((rc = vec_f32(e, m, a + "k.norm", d.head_dim, 1, &L.k_norm))) return rc;
            if ((rc = matrix(e, a + "o", W, qd, L.attn_o))) return rc;
            if ((rc = vec_f32(e, m, a + "out", W, 1, &L.left_w))) return rc;
            if ((rc = vec_f32(e, m, b + "out", W, 1, &L.right_w))) return rc;
            if ((rc = vec_f32(e, m, b + "conv", d.conv_taps, d.d_inner, &L.conv_w))) return rc;
            if ((rc = vec_f32(e, m, b + "conv.b", d.d_inner, 1, &L.conv_b))) return rc;
            if ((rc = matrix(e, b + "x", d.dt_rank + 2 * d.d_state, d.d_inner, L.scan_x))) return rc;
            if ((rc = matrix(e, b + "dt", d.d_inner, d.dt_rank, L.scan_dt))) return rc;
            if ((rc = vec_f32(e, m, b + "dt.b", d.d_inner, 1, &L.dt_b))) return rc;
            if ((rc = vec_f32(e, m, b + "A_log", d.d_state, d.d_inner, &L.A_log))) return rc;
            if ((rc = vec_f32(e, m, b + "D", d.d_inner, 1, &L.Dskip))) return rc;
            if ((rc = matrix(e, b + "o", W, d.d_inner, L.scan_o))) return rc;
            if ((rc = build_rotary(e, m, L))) return rc;
            const size_t pool = (size_t)c.kv_num_blocks * d.n_head_kv * c.kv_block_tokens * d.head_dim * cache_esz;
            if ((rc = dev_alloc(m, &L.k_pool, pool, true))) return rc;
            if ((rc = dev_alloc(m, &L.v_pool, pool, true))) return rc;
            e->kv_bytes += 2 * (int64_t)pool;
            if ((rc = dev_alloc(m, (void**)&L.conv_state, (size_t)S * d.d_inner * std::max(1, d.conv_taps - 1) * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.ssm_state, (size_t)S * d.d_inner * d.d_state * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.in_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)qd, (size_t)d.d_inner, (size_t)d.dt_rank + 2 * d.d_state});
            max_attn = 1; max_attn_d = std::max<size_t>(max_attn_d, d.head_dim);
        } else {
            const std::string a = p + "mix.";
            const int qd = d.mm_heads * d.mm_dim, vd = d.mm_heads * d.mm_vdim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", qd}, {a + "k", qd}, {a + "v", vd}, {a + "g", vd}, {a + "i", d.mm_heads}, {a + "f", d.mm_heads}}, W, L.mm_proj, offs))) return rc;
            L.mq = offs[0]; L.mk = offs[1]; L.mv = offs[2]; L.mg = offs[3]; L.mi = offs[4]; L.mf = offs[5];
            if ((rc = vec_f32(e, m, a + "i.b", d.mm_heads, 1, &L.i_b))) return rc;
            if ((rc = vec_f32(e, m, a + "f.b", d.mm_heads, 1, &L.f_b))) return rc;
            if ((rc = vec_f32(e, m, a + "norm", vd, 1, &L.mm_norm))) return rc;
            if ((rc = matrix(e, a + "o", W, vd, L.mm_o))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.S, (size_t)S * d.mm_heads * d.mm_dim * d.mm_vdim * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.nvec, (size_t)S * d.mm_heads * d.mm_dim * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.mmax, (size_t)S * d.mm_heads * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.mm_proj.N);
            max_buf = std::max<size_t>(max_buf, (size_t)vd);
        }
        if (d.n_ff > 0) {
            if ((rc = vec_f32(e, m, p + "norm2", W, 1, &L.norm2))) return rc;
            if ((rc = matrix(e, p + "mlp.up", d.n_ff, W, L.up))) return rc;
            if ((rc = vec_f32(e, m, p + "mlp.up.b", d.n_ff, 1, &L.up_b))) return rc;
            if ((rc = matrix(e, p + "mlp.down", W, d.n_ff, L.down))) return rc;
            if ((rc = vec_f32(e, m, p + "mlp.down.b", W, 1, &L.down_b))) return rc;
            max_ff = std::max<size_t>(max_ff, d.n_ff);
        }
    }
    if ((rc = dev_alloc(m, (void**)&m->x, (size_t)Tm * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->proj, (size_t)Tm * max_proj * 4))) return rc;
    for (int i = 0; i < 4; i++) if ((rc = dev_alloc(m, (void**)&m->buf[i], (size_t)Tm * max_buf * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->oL, (size_t)Tm * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->oR, (size_t)Tm * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->ff, (size_t)Tm * max_ff * 4))) return rc;
    if (!m->exact && (rc = dev_alloc(m, (void**)&m->xb, (size_t)(Tm + B2_STEP_MAX_ENTRIES) * std::max<size_t>({max_buf, max_ff, (size_t)W}) * 2 + 64))) return rc;
    if (max_attn > 0) {
        m->attn_split_floats = (int)(148 * 2 * (max_attn_d + 2));       // T * H * splits <= 2 * 148 on the split path
        if ((rc = dev_alloc(m, (void**)&m->attn_split, (size_t)m->attn_split_floats * 4))) return rc;
    }
    if ((rc = dev_alloc(m, (void**)&m->rows, (size_t)LOGIT_ROWS * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->logits, (size_t)LOGIT_ROWS * V * 4))) return rc;
    const size_t n_meta = (size_t)4 * Tm + 2 * (Tm / 64 + B2_STEP_MAX_ENTRIES) + 5 * B2_STEP_MAX_ENTRIES + 64;
    if ((rc = dev_alloc(m, (void**)&m->meta, n_meta * 4))) return rc;
    CK(cudaMallocHost(&m->meta_host, n_meta * 4));
    CK(cudaMallocHost(&m->logits_host, (size_t)LOGIT_ROWS * V * 4));
    {
        std::vector<int*> tabs(S);
        for (int i = 0; i < S; i++) tabs[i] = e->slots[i].block_table;
        if ((rc = dev_alloc(m, (void**)&m->block_tables, sizeof(int*) * S))) return rc;
        CK(cudaMemcpy(m->block_tables, tabs.data(), sizeof(int*) * S, cudaMemcpyHostToDevice));
    }
    CK(cudaStreamSynchronize(e->stream));
    e->finalized = true;
    return B2_OK;
}

void layered_destroy(b2_engine* e) {
    LayeredModel* m = e->layered;
    if (!m) return;
    for (void* p : m->owned) cudaFree(p);
    if (m->meta_host) cudaFreeHost(m->meta_host);
    if (m->logits_host) cudaFreeHost(m->logits_host);
    for (auto& pe : m->prof_ev) { cudaEventDestroy(pe.second.first); cudaEventDestroy(pe.second.second); }
    for (auto& kv : m->graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    delete m;
    e->layered = nullptr;
}

// a slot starts a new sequence: its recurrent state goes back to zero (cache pages are simply overwritten)
int layered_seq_reset(b2_engine* e, int slot) {
    LayeredModel* m = e->layered;
    for (auto& L : m->layers) {
        const b2_layer_desc& d = L.d;
        if (d.mixer == B2_MIX_WINDOW_SCAN) {
            const size_t cs = (size_t)d.d_inner * std::max(1, d.conv_taps - 1), ss = (size_t)d.d_inner * d.d_state;
            CK(cudaMemsetAsync(L.conv_state + slot * cs, 0, cs * 4, e->stream));
            CK(cudaMemsetAsync(L.ssm_state + slot * ss, 0, ss * 4, e->stream));
        } else {
            const size_t s1 = (size_t)d.mm_heads * d.mm_dim * d.mm_vdim, s2 = (size_t)d.mm_heads * d.mm_dim;
            CK(cudaMemsetAsync(L.S + slot * s1, 0, s1 * 4, e->stream));
            CK(cudaMemsetAsync(L.nvec + slot * s2, 0, s2 * 4, e->stream));
            CK(cudaMemsetAsync(L.mmax + slot * d.mm_heads, 0, (size_t)d.mm_heads * 4, e->stream));
        }
    }
    return B2_OK;
}

}  // namespace b2

// ------------------------------------------------------------------------------------------ C ABI
extern "C" int b2_engine_create_layered(const b2_layered_config* c, const b2_layer_desc* layers, b2_engine** out) {
    if (!c || !layers || !out) return b2_fail(B2_ERR_ARG, "null argument");
    if (c->n_layer <= 0 || c->n_embd <= 0 || c->n_vocab <= 0 || c->n_ctx <= 0 || c->max_seqs <= 0 || c->kv_block_tokens <= 0 ||
        c->kv_num_blocks <= 0 || c->max_step_tokens <= 0)
        return b2_fail(B2_ERR_ARG, "bad model/config dimensions");
    if (c->max_seqs > B2_STEP_MAX_ENTRIES) return b2_fail(B2_ERR_ARG, "at most 64 sequence slots");
    for (int i = 0; i < c->n_layer; i++) {
        const b2_layer_desc& d = layers[i];
        const std::string li = "layer " + std::to_string(i) + ": ";
        if (d.n_ff < 0) return b2_fail(B2_ERR_ARG, li + "negative feed-forward width");
        if (d.mixer == B2_MIX_WINDOW_SCAN) {
            if (d.n_head <= 0 || d.n_head_kv <= 0 || d.n_head % d.n_head_kv || d.head_dim <= 0) return b2_fail(B2_ERR_ARG, li + "bad head counts");
            if (d.head_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "head size above 256");
            if (d.rot_dims < 0 || d.rot_dims > d.head_dim || d.rot_dims % 2) return b2_fail(B2_ERR_ARG, li + "rotary dims must be even and <= the head size");
            if (d.window <= 0 || d.keep_first < 0) return b2_fail(B2_ERR_ARG, li + "bad window");
            if (d.conv_taps <= 0 || d.conv_taps > 64 || d.dt_rank <= 0 || d.d_inner <= 0 || d.d_state <= 0) return b2_fail(B2_ERR_ARG, li + "bad scan sizes");
            if (d.d_state > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "scan state above 256");
        } else if (d.mixer == B2_MIX_MATRIX_MEMORY) {
            if (d.mm_heads <= 0 || d.mm_dim <= 0 || d.mm_vdim <= 0 || !(d.gate_cap > 0.0)) return b2_fail(B2_ERR_ARG, li + "bad matrix-memory sizes");
            if (d.mm_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "matrix-memory key size above 256");
        } else return b2_fail(B2_ERR_UNSUPPORTED, li + "unknown mixer kind");
    }
    b2_engine* e = new b2_engine();
    b2_config& b = e->cfg;
    memset(&b, 0, sizeof(b));
    b.n_layer = c->n_layer; b.n_embd = c->n_embd; b.n_vocab = c->n_vocab; b.rms_eps = c->norm_eps; b.n_ctx = c->n_ctx;
    b.max_seqs = c->max_seqs; b.kv_block_tokens = c->kv_block_tokens; b.kv_num_blocks = c->kv_num_blocks; b.device = c->device;
    b.flags = c->flags;
    LayeredModel* m = new LayeredModel();
    m->c = *c;
    m->exact = (c->flags & B2_FLAG_F32) != 0;
    m->layers.resize(c->n_layer);
    for (int i = 0; i < c->n_layer; i++) m->layers[i].d = layers[i];
    e->layered = m;
    e->use_graph = !(c->flags & B2_FLAG_NO_GRAPH) && !getenv("B2_NO_GRAPH");
    m->graphs_on = e->use_graph;
    e->use_pdl = e->chain_pdl = !(c->flags & B2_FLAG_NO_PDL) && !getenv("B2_NO_CHAIN_PDL");
    auto init = [&]() -> int {
        CK(cudaSetDevice(c->device));
        cudaDeviceGetAttribute(&e->n_sms, cudaDevAttrMultiProcessorCount, c->device);
        CK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
        CK(cudaEventCreate(&e->ev0));
        CK(cudaEventCreate(&e->ev1));
        CK(cudaMallocHost(&e->pinned, sizeof(int32_t) * (size_t)(c->max_seqs + B2_STEP_MAX_ENTRIES + 16)));
        e->max_blocks = (c->n_ctx + c->kv_block_tokens - 1) / c->kv_block_tokens;
        e->slots.resize(c->max_seqs);
        for (auto& s : e->slots) {
            CK(cudaMalloc(&s.logits, sizeof(float) * c->n_vocab));
            CK(cudaMalloc(&s.ints, sizeof(int) * 8));
            CK(cudaMemset(s.ints, 0, sizeof(int) * 8));
            CK(cudaMalloc(&s.block_table, sizeof(int) * e->max_blocks));
            CK(cudaMemset(s.block_table, 0, sizeof(int) * e->max_blocks));
            CK(cudaMalloc(&s.ring, sizeof(int) * (c->n_ctx + 1)));
            CK(cudaMemset(s.ring, 0, sizeof(int) * (c->n_ctx + 1)));
            CK(cudaMalloc(&s.sst, sizeof(SamplerState)));
            CK(cudaMemset(s.sst, 0, sizeof(SamplerState)));
            CK(cudaMalloc(&s.sp, sizeof(SampleParams)));
            CK(cudaMemset(s.sp, 0, sizeof(SampleParams)));
            CK(cudaMalloc(&s.uniforms, sizeof(double) * 8192));
            CK(cudaMemset(s.uniforms, 0, sizeof(double) * 8192));
        }
        return B2_OK;
    };
    const int rc = init();
    if (rc) { b2_engine_destroy(e); return rc; }
    *out = e;
    return B2_OK;
}

namespace {
struct StepProfiler {                 // events around launches of one kind, only when profiling is on
    LayeredModel* m; cudaStream_t st; cudaEvent_t b = nullptr;
    int kind;
    StepProfiler(LayeredModel* m_, cudaStream_t s, int k) : m(m_), st(s), kind(k) {
        if (!m->profile) return;
        cudaEvent_t a; cudaEventCreate(&a); cudaEventCreate(&b);
        cudaEventRecord(a, st);
        m->prof_ev.push_back({kind, {a, b}});
    }
    ~StepProfiler() { if (b) cudaEventRecord(b, st); }
};
}  // namespace

static int dense(b2_engine* e, LayeredModel* m, const DenseW& w, const float* x, int ldx, float* y, int ldy, int T,
                 const float* bias = nullptr, int epi = EPI_NONE, int kind = 1) {
    StepProfiler sp(m, e->stream, kind);
    DenseArgs a = {};
    a.x = x; a.ldx = ldx; a.w = w.w; a.w_type = w.type; a.bias = bias; a.y = y; a.ldy = ldy; a.T = T; a.N = w.N; a.K = w.K;
    a.epi = epi; a.exact = m->exact; a.xb = m->xb;
    CK(dense_launch(a, e->stream));
    e->launches++;
    return B2_OK;
}

static int run_layers(b2_engine* e, LayeredModel* m, const RaggedDev& r) {
    const b2_layered_config& c = m->c;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd;
    int rc;
    {
        StepProfiler sp(m, st, 0);
        CK(embed_ragged_launch(m->embed.w, m->embed.type, W, r.tok_id, T, m->x, st));
        e->launches++;
    }
    for (int li = 0; li < c.n_layer; li++) {
        LyLayer& L = m->layers[li];
        const b2_layer_desc& d = L.d;
        if (d.mixer == B2_MIX_WINDOW_SCAN) {
            const int Np = L.in_proj.N, qd = d.n_head * d.head_dim;
            if ((rc = dense(e, m, L.in_proj, m->x, W, m->proj, Np, T))) return rc;
            WindowAttnArgs a = {};
            a.proj = m->proj; a.ldp = Np; a.q_off = L.q_off; a.k_off = L.k_off; a.q_norm_w = L.q_norm; a.k_norm_w = L.k_norm;
            a.rot.cos = L.rot_cos; a.rot.sin = L.rot_sin; a.rot.rot_dims = d.rot_dims;
            a.k_pool = L.k_pool; a.v_pool = L.v_pool; a.cache_f32 = m->exact ? 1 : 0; a.block_tables = m->block_tables;
            a.block_tokens = c.kv_block_tokens; a.H = d.n_head; a.G = d.n_head_kv; a.d = d.head_dim; a.window = d.window;
            a.keep_first = d.keep_first; a.scale = (float)d.attn_scale; a.eps = c.norm_eps; a.q_rot = m->buf[0]; a.out = m->buf[1];
            a.split_scratch = m->attn_split; a.split_capacity = m->attn_split_floats;
            {
                StepProfiler sp(m, st, 2);
                CK(window_attn_store_launch(a, r, st));
                CK(window_attn_launch(a, r, st));
                e->launches += 2;
            }
            if ((rc = dense(e, m, L.attn_o, m->buf[1], qd, m->oL, W, T))) return rc;
            ScanArgs s = {};
            s.proj = m->proj; s.ldp = Np; s.x_off = L.x_off; s.z_off = L.z_off; s.conv_w = L.conv_w; s.conv_b = L.conv_b;
            s.taps = d.conv_taps; s.conv_state = L.conv_state; s.xc = m->buf[0]; s.xproj = m->buf[2];
            s.ldx = d.dt_rank + 2 * d.d_state; s.R = d.dt_rank; s.N = d.d_state; s.dt_raw = m->buf[3]; s.dt_bias = L.dt_b;
            s.A_log = L.A_log; s.D = L.Dskip; s.ssm_state = L.ssm_state; s.y = m->buf[1]; s.inner = d.d_inner;
            {
                StepProfiler sp(m, st, 3);
                CK(scan_conv_launch(s, r, st));
                e->launches++;
            }
            if ((rc = dense(e, m, L.scan_x, m->buf[0], d.d_inner, m->buf[2], s.ldx, T))) return rc;
            if ((rc = dense(e, m, L.scan_dt, m->buf[2], s.ldx, m->buf[3], d.d_inner, T))) return rc;
            {
                StepProfiler sp(m, st, 3);
                CK(scan_recurrence_launch(s, r, st));
                e->launches += d.d_state <= 32 ? 2 : 1;      // states up to a warp wide: a preparation pass goes first
            }
            if ((rc = dense(e, m, L.scan_o, m->buf[1], d.d_inner, m->oR, W, T))) return rc;
            StepProfiler sp(m, st, 5);
            CK(postsum_norm_launch(m->x, m->oL, L.left_w, m->oR, L.right_w, L.norm1, c.residual_scale, c.norm_eps, W, T, st));
            e->launches++;
        } else {
            const int Np = L.mm_proj.N, vd = d.mm_heads * d.mm_vdim;
            if ((rc = dense(e, m, L.mm_proj, m->x, W, m->proj, Np, T))) return rc;
            MatrixMemArgs a = {};
            a.proj = m->proj; a.ldp = Np; a.q_off = L.mq; a.k_off = L.mk; a.v_off = L.mv; a.g_off = L.mg; a.i_off = L.mi; a.f_off = L.mf;
            a.i_bias = L.i_b; a.f_bias = L.f_b; a.norm_w = L.mm_norm; a.H = d.mm_heads; a.d = d.mm_dim; a.dv = d.mm_vdim;
            a.cap = (float)d.gate_cap; a.eps = c.norm_eps; a.S = L.S; a.n = L.nvec; a.m = L.mmax; a.o_raw = m->buf[0]; a.out = m->buf[1];
            {
                StepProfiler sp(m, st, 4);
                CK(matrix_mem_launch(a, r, st));
                e->launches += 3;
            }
            if ((rc = dense(e, m, L.mm_o, m->buf[1], vd, m->oL, W, T))) return rc;
            StepProfiler sp(m, st, 5);
            CK(postsum_norm_launch(m->x, m->oL, nullptr, nullptr, nullptr, L.norm1, c.residual_scale, c.norm_eps, W, T, st));
            e->launches++;
        }
        if (d.n_ff > 0) {
            if ((rc = dense(e, m, L.up, m->x, W, m->ff, d.n_ff, T, L.up_b, EPI_BIAS_RELU2))) return rc;
            if ((rc = dense(e, m, L.down, m->ff, d.n_ff, m->oL, W, T, L.down_b, EPI_BIAS))) return rc;
            StepProfiler sp(m, st, 5);
            CK(postsum_norm_launch(m->x, m->oL, nullptr, nullptr, nullptr, L.norm2, c.residual_scale, c.norm_eps, W, T, st));
            e->launches++;
        }
        if (m->trace)
            CK(cudaMemcpyAsync(m->trace + ((size_t)li * c.max_step_tokens) * W, m->x, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st));
    }
    return B2_OK;
}

struct StepChainPdl {
    bool prev;
    explicit StepChainPdl(bool on) : prev(g_chain_pdl) { g_chain_pdl = on; }
    ~StepChainPdl() { g_chain_pdl = prev; }
};

int b2_sample_enqueue(b2_engine* e, Slot& s, int pinned_index);

extern "C" int b2_step(b2_engine* e, int n_entries, const int32_t* slots, const int32_t* n_tokens, const int32_t* tokens,
                       const int32_t* want_rows, int n_want, float* host_logits, const int32_t* sample, int32_t* host_sampled) {
    if (!e || !e->layered) return b2_fail(B2_ERR_UNSUPPORTED, "b2_step needs an engine made by b2_engine_create_layered");
    if (!e->finalized) return b2_fail(B2_ERR_STATE, "engine not finalized");
    if (n_entries <= 0 || n_entries > B2_STEP_MAX_ENTRIES || !slots || !n_tokens || !tokens) return b2_fail(B2_ERR_ARG, "bad arguments");
    if (n_want < 0 || (n_want > 0 && (!want_rows || !host_logits))) return b2_fail(B2_ERR_ARG, "bad wanted rows");
    std::lock_guard<std::mutex> lk(e->mu);
    LayeredModel* m = e->layered;
    const b2_layered_config& c = m->c;
    int T = 0;
    for (int i = 0; i < n_entries; i++) {
        if (slots[i] < 0 || slots[i] >= c.max_seqs) return b2_fail(B2_ERR_ARG, "slot out of range");
        for (int j = 0; j < i; j++) if (slots[j] == slots[i]) return b2_fail(B2_ERR_ARG, "slot listed twice");
        if (n_tokens[i] <= 0) return b2_fail(B2_ERR_ARG, "empty entry");
        if (e->slots[slots[i]].n_past + n_tokens[i] > c.n_ctx) return b2_fail(B2_ERR_ARG, "context window full");
        T += n_tokens[i];
        if (T > c.max_step_tokens) return b2_fail(B2_ERR_ARG, "more tokens than max_step_tokens in one step");
    }
    for (int i = 0; i < T; i++) if (tokens[i] < 0 || tokens[i] >= c.n_vocab) return b2_fail(B2_ERR_ARG, "token id out of range");
    for (int i = 0; i < n_want; i++) if (want_rows[i] < 0 || want_rows[i] >= T) return b2_fail(B2_ERR_ARG, "wanted row out of range");
    CK(cudaSetDevice(c.device));
    cudaStream_t st = e->stream;
    StepChainPdl chain(e->chain_pdl);
    // ragged description: [tok_id T][tok_seg T][tok_pos T][seg_slot n][seg_start n][seg_len n][seg_pos0 n][tile_seg][tile_row0][rows ...]
    int* h = m->meta_host;
    const int n = n_entries;
    int *h_id = h, *h_seg = h + T, *h_pos = h + 2 * T, *h_slot = h + 3 * T, *h_start = h_slot + n, *h_len = h_start + n, *h_p0 = h_len + n;
    int n_tiles = 0;
    for (int i = 0; i < n; i++) n_tiles += (n_tokens[i] + 63) / 64;
    int *h_tseg = h_p0 + n, *h_trow = h_tseg + n_tiles;
    int* h_rows = h_trow + n_tiles;
    int row = 0, tile = 0;
    for (int i = 0; i < n; i++) {
        const int p0 = e->slots[slots[i]].n_past;
        h_slot[i] = slots[i]; h_start[i] = row; h_len[i] = n_tokens[i]; h_p0[i] = p0;
        for (int k = 0; k < n_tokens[i]; k += 64) { h_tseg[tile] = i; h_trow[tile++] = row + k; }
        for (int k = 0; k < n_tokens[i]; k++, row++) { h_id[row] = tokens[row]; h_seg[row] = i; h_pos[row] = p0 + k; }
    }
    // rows whose logits are needed: the wanted ones, then the last token of every sampled entry
    int n_rows = 0;
    for (int i = 0; i < n_want; i++) h_rows[n_rows++] = want_rows[i];
    std::vector<int> samp_row(n, -1);
    for (int i = 0; i < n; i++)
        if (sample && sample[i]) { samp_row[i] = n_rows; h_rows[n_rows++] = h_start[i] + h_len[i] - 1; }
    const size_t n_meta = (size_t)3 * T + 4 * n + 2 * n_tiles + n_rows;
    RaggedDev r = {};
    r.tok_id = m->meta; r.tok_seg = m->meta + T; r.tok_pos = m->meta + 2 * T; r.seg_slot = m->meta + 3 * T;
    r.seg_start = r.seg_slot + n; r.seg_len = r.seg_start + n; r.seg_pos0 = r.seg_len + n; r.T = T; r.n_seg = n;
    r.tile_seg = r.seg_pos0 + n; r.tile_row0 = r.tile_seg + n_tiles; r.n_tiles = n_tiles;
    const int* d_rows = r.tile_row0 + n_tiles;
    if (m->profile) {
        for (auto& pe : m->prof_ev) { cudaEventDestroy(pe.second.first); cudaEventDestroy(pe.second.second); }
        m->prof_ev.clear();
    }
    const int W = c.n_embd, V = c.n_vocab;
    int rc;
    // logits of rows [r0, r0 + nr): final norm, head, wanted rows to the pinned buffer, sampled rows to their slots
    auto head_chunk = [&](int r0, int nr) -> int {
        {
            StepProfiler sp(m, st, 5);
            CK(gather_rows_launch(m->x, W, d_rows + r0, nr, m->rows, st));
            CK(layer_norm_launch(m->rows, m->final_norm, c.norm_eps, W, nr, m->rows, st));
            e->launches += 2;
        }
        int rc2 = dense(e, m, m->head, m->rows, W, m->logits, V, nr, nullptr, EPI_NONE, 6);
        if (rc2) return rc2;
        const int n_w = std::max(0, std::min(n_want - r0, nr));
        if (n_w > 0) CK(cudaMemcpyAsync(m->logits_host, m->logits, (size_t)n_w * V * 4, cudaMemcpyDeviceToHost, st));
        for (int i = 0; i < n; i++)
            if (samp_row[i] >= r0 && samp_row[i] < r0 + nr)
                CK(cudaMemcpyAsync(e->slots[slots[i]].logits, m->logits + (size_t)(samp_row[i] - r0) * V, (size_t)V * 4, cudaMemcpyDeviceToDevice, st));
        return B2_OK;
    };
    // everything the step enqueues up to the logits, for steps whose rows fit one head chunk
    auto forward_once = [&]() -> int {
        CK(cudaMemcpyAsync(m->meta, h, n_meta * 4, cudaMemcpyHostToDevice, st));
        int rc2 = run_layers(e, m, r);
        if (rc2) return rc2;
        return n_rows > 0 ? head_chunk(0, n_rows) : B2_OK;
    };
    // Small steps that repeat (the same slots decoding token after token) are replayed as a CUDA graph: the batch description
    // is read from device memory, so nothing in the launches changes from one such step to the next. A shape is captured the
    // second time it is seen.
    bool done = false;
    if (m->graphs_on && !m->trace && !m->profile && T <= 64 && n_rows <= LOGIT_ROWS) {
        std::string key;
        key.reserve(16 + 12 * n);
        auto put = [&](int v) { key.append(reinterpret_cast<const char*>(&v), sizeof(v)); };
        put(n); put(n_want);
        for (int i = 0; i < n; i++) { put(slots[i]); put(n_tokens[i]); put(samp_row[i]); }
        auto it = m->graphs.find(key);
        if (it == m->graphs.end()) {
            if (m->graphs.size() >= 256) {
                for (auto& kv : m->graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
                m->graphs.clear();
            }
            m->graphs[key] = StepGraph();
        } else {
            StepGraph& sg = it->second;
            if (!sg.exec && !sg.failed) {
                const int64_t before = e->launches;
                cudaGraph_t g = nullptr;
                CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
                const int crc = forward_once();
                const cudaError_t ce = cudaStreamEndCapture(st, &g);
                sg.n_launch = (int)(e->launches - before);
                e->launches = before;
                if (crc == B2_OK && ce == cudaSuccess && g && cudaGraphInstantiate(&sg.exec, g, 0) != cudaSuccess) sg.exec = nullptr;
                if (g) cudaGraphDestroy(g);
                if (!sg.exec) { sg.failed = true; cudaGetLastError(); }
            }
            if (sg.exec) {
                CK(cudaGraphLaunch(sg.exec, st));
                e->launches += sg.n_launch;
                done = true;
            }
        }
    }
    if (!done) {
        if (n_rows <= LOGIT_ROWS) {
            if ((rc = forward_once())) return rc;
        } else {
            CK(cudaMemcpyAsync(m->meta, h, n_meta * 4, cudaMemcpyHostToDevice, st));
            if ((rc = run_layers(e, m, r))) return rc;
        }
    }
    m->last_T = T;
    for (int i = 0; i < n; i++) if (samp_row[i] >= 0) e->slots[slots[i]].logits_view = e->slots[slots[i]].logits;
    if (n_rows <= LOGIT_ROWS) {
        if (n_want > 0) {
            CK(cudaStreamSynchronize(st));
            memcpy(host_logits, m->logits_host, (size_t)n_want * V * 4);
        }
    } else {
        for (int r0 = 0; r0 < n_rows; r0 += LOGIT_ROWS) {
            const int nr = std::min(LOGIT_ROWS, n_rows - r0);
            if ((rc = head_chunk(r0, nr))) return rc;
            const int n_w = std::max(0, std::min(n_want - r0, nr));
            if (n_w > 0) {
                CK(cudaStreamSynchronize(st));
                memcpy(host_logits + (size_t)r0 * V, m->logits_host, (size_t)n_w * V * 4);
            }
        }
    }
    for (int i = 0; i < n; i++) e->slots[slots[i]].n_past += n_tokens[i];
    for (int i = 0; i < n; i++) {
        if (host_sampled) host_sampled[i] = -1;
        if (samp_row[i] >= 0) { if ((rc = b2_sample_enqueue(e, e->slots[slots[i]], i))) return rc; }
    }
    CK(cudaStreamSynchronize(st));
    if ((rc = b2_check_kernel_error())) return rc;
    if (host_sampled) for (int i = 0; i < n; i++) if (samp_row[i] >= 0) host_sampled[i] = e->pinned[i];
    if (m->profile) {
        for (int k = 0; k < 8; k++) { m->prof_ms[k] = 0.f; m->prof_n[k] = 0; }
        for (auto& pe : m->prof_ev) {
            float t = 0.f;
            cudaEventElapsedTime(&t, pe.second.first, pe.second.second);
            m->prof_ms[pe.first] += t; m->prof_n[pe.first]++;
        }
    }
    return B2_OK;
}

extern "C" int b2_step_trace(b2_engine* e, int on) {
    if (!e || !e->layered) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    LayeredModel* m = e->layered;
    CK(cudaSetDevice(m->c.device));
    if (on && !m->trace) {
        int rc = dev_alloc(m, (void**)&m->trace, (size_t)m->c.n_layer * m->c.max_step_tokens * m->c.n_embd * 4);
        if (rc) return rc;
    }
    if (!on) m->trace = nullptr;       // the buffer stays owned and is freed with the engine
    return B2_OK;
}

extern "C" int b2_step_trace_read(b2_engine* e, float* out, int n_layer, int T) {
    if (!e || !e->layered || !out) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    LayeredModel* m = e->layered;
    if (!m->trace) return b2_fail(B2_ERR_STATE, "tracing is off");
    if (n_layer != m->c.n_layer || T != m->last_T) return b2_fail(B2_ERR_ARG, "shape does not match the last step");
    CK(cudaSetDevice(m->c.device));
    const size_t W = m->c.n_embd;
    for (int l = 0; l < n_layer; l++)
        CK(cudaMemcpy(out + (size_t)l * T * W, m->trace + (size_t)l * m->c.max_step_tokens * W, (size_t)T * W * 4, cudaMemcpyDeviceToHost));
    return B2_OK;
}

extern "C" int b2_step_profile(b2_engine* e, int on) {
    if (!e || !e->layered) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    e->layered->profile = on != 0;
    return B2_OK;
}

extern "C" int b2_step_profile_read(b2_engine* e, float* ms, int32_t* nl) {
    if (!e || !e->layered || !ms || !nl) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    for (int k = 0; k < 8; k++) { ms[k] = e->layered->prof_ms[k]; nl[k] = e->layered->prof_n[k]; }
    return B2_OK;
}
