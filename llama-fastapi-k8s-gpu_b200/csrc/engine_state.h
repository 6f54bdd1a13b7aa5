// Engine object shared by the model graphs (engine.cu: the llama graph over GGUF blocks; layered.cu: the layer-list
// graph over dense bf16/f32 tensors) and the error plumbing of the C ABI. Internal: the public surface is
// include/b200_gguf.h.
#pragma once
#include "../../include/b200_gguf.h"
#include "kernels.h"

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

// records the message b2_last_error() returns on this thread and passes the code through
int b2_fail(int code, const std::string& msg);
// kernel watchdogs report through a host-mapped word; call after a synchronise
int b2_check_kernel_error();
#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t _e = (call);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return b2_fail(B2_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_e));      \
    } while (0)

namespace b2 { struct LayeredModel; }
using namespace b2;

struct DevTensor {
    uint8_t* ptr = nullptr;
    int type = -1;
    int64_t ne0 = 0, ne1 = 0, nbytes = 0;
};

struct Layer {
    DevTensor attn_norm, wq, wk, wv, wo, ffn_norm, wgate, wup, wdown;
    MvParams p_qkv, p_o, p_gu, p_down;
    MvParams p_gate, p_up;         // un-fused pair when ffn_gate and ffn_up have different quant types
    bool gu_fused = true;
};

struct Slot {
    float *x = nullptr, *q = nullptr, *att = nullptr, *h = nullptr, *hg = nullptr, *logits = nullptr;
    float* tp_part = nullptr;      // tensor parallelism: this rank's partial sum of attn_output / ffn_down (rank 0: + the residual)
    int* ints = nullptr;           // [0]=token [1]=pos [2]=out_token [3]=step [4]=cursor [5]=pos_base
    int* block_table = nullptr;
    int* prompt = nullptr;         // [n_ctx]
    int* ring = nullptr;           // [n_ctx + 1] sampled token by position
    SamplerState* sst = nullptr;
    SampleParams* sp = nullptr;
    double* uniforms = nullptr;    // [8192]
    cudaGraphExec_t g_decode = nullptr, g_pre_step = nullptr, g_pre_last = nullptr, g_fwd = nullptr;
    int n_decode_nodes = 0, n_pre_step_nodes = 0, n_pre_last_nodes = 0, n_fwd_nodes = 0;
    const float* logits_view = nullptr;   // where the latest logits of this slot are (own buffer, or a row of the batch output)
    int n_past = 0;                // host mirror of ints[1]
    int n_sampled = 0;             // host mirror of ints[3]
};

struct b2_engine {
    b2_config cfg;
    cudaStream_t stream = nullptr;
    std::unordered_map<std::string, DevTensor> tensors;
    std::vector<Layer> layers;
    DevTensor tok_embd, out_norm, output;
    MvParams p_head;
    __half *k_pool = nullptr, *v_pool = nullptr;
    size_t layer_kv_elems = 0;
    float* rope_freq = nullptr;
    float* attn_scratch = nullptr;
    unsigned* attn_counters = nullptr;
    int n_splits = 1, max_blocks = 0, n_ctas = 148;
    std::vector<Slot> slots;
    int32_t* pinned = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int64_t launches = 0, weight_bytes = 0, kv_bytes = 0;
    bool use_graph = true, use_pdl = true, act2 = true, finalized = false, chain_pdl = true;
    int batch_attn_splits = 0;     // B2_BATCH_ATTN_SPLITS (tuning), read once at create
    int attn_early = 1;            // B2_ATTN_EARLY=0 (tuning): attention requests nothing before its dependency wait
    // tensor parallelism (b2_engine_tp_init): this engine holds 1 / tp_world of the heads, FFN rows and vocabulary rows
    void* tp_comm = nullptr;
    int tp_rank = 0, tp_world = 1;
    // all-reduce over peer memory (tp.cu): [2][n_embd] partial sums + flags + sequence number in one IPC-shared allocation
    float* tp_shared = nullptr;
    void* tp_peer[TP_MAX_WORLD] = {};
    bool tp_p2p = false;
    TpArParams tp_ar[2] = {};
    unsigned long long* tl = nullptr;   // B2_TIMELINE=1: 4 time stamps per kernel of a decode step (debugging aid)
    int tl_n = 0;                  // kernels recorded by the last forward_launches
    // prompt (GEMM) workspace, allocated on the first long prompt: PF_T tokens per chunk
    float *pf_x = nullptr, *pf_part = nullptr;     // residual stream [PF_T][n_embd]; K-split partial sums of the last GEMM
    size_t pf_part_floats = 0;
    __half *pf_xn = nullptr, *pf_qh = nullptr, *pf_att = nullptr, *pf_h = nullptr;
    int n_sms = 148;
    // batched decode (several sequences per step through the GEMM path)
    SlotDev* slot_tab = nullptr;   // device table, one entry per slot
    float *bd_q = nullptr, *bd_att = nullptr, *bd_scratch = nullptr;
    unsigned* bd_counters = nullptr;
    int* bd_out = nullptr;
    int attn_mma = -1;             // tensor-core flash-decode: -1 = batched steps only; 0 never; 1 always
    int batch_min = 3;             // fewer sequences than this step one after another through the mat-vec path (measured: 3 slots 4.1 vs 6.3 ms)
    bool gemm_ok = false;          // every layer matrix is a block format the GEMM reads
    int prefill_min = 8;           // prompts chunks shorter than this go token by token through the mat-vec path
    // GEMM launch plans (tile split, K splits, tensor maps) are built once per (first weight matrix, token count) and reused:
    // re-planning -- cuTensorMapEncodeTiled and a handful of getenv per call -- for each of the 129 GEMMs of every batched
    // step cost more host time than the step takes on the GPU
    std::unordered_map<uint64_t, GemmParams> gemm_plans;
    // layer-list models (b2_engine_create_layered): graph, dense weights, KV pools and recurrent state live here
    LayeredModel* layered = nullptr;
    std::mutex mu;
};

