// Host side of libwick_cuda: GGUF -> device model, the decode / prefill drivers
// and the C ABI of include/wick_cuda.h.  The structure follows the role
// MetalLfm2Model plays in wick (wick/src/model/metal_lfm2.rs:170-277, :280-610):
// one sequence lives in the model; weights, KV cache, conv state and scratch are
// device resident; a decode step is one submission (here: one CUDA graph launch).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <initializer_list>
#include <memory>
#include <string>
#include <vector>

#include "../../include/wick_cuda.h"
#include "gguf.hpp"
#include "decode_mega.cuh"
#include "gemm_tc.cuh"
#include "kernels.cuh"

using namespace wick;

// ── errors ─────────────────────────────────────────────────────────────────
static thread_local std::string g_last_error;

static int32_t fail(int32_t code, const std::string& msg) {
    g_last_error = msg;
    return code;
}
#define CU_TRY(expr)                                                                              \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess)                                                                   \
            return fail(e__ == cudaErrorMemoryAllocation ? WICK_CUDA_ERR_OOM : WICK_CUDA_ERR_CUDA, \
                        std::string(#expr) + ": " + cudaGetErrorString(e__));                     \
    } while (0)
#define W_TRY(expr)                  \
    do {                             \
        int32_t r__ = (expr);        \
        if (r__ != WICK_CUDA_OK) return r__; \
    } while (0)

namespace {

struct Layer {
    bool is_attn = false;
    int n_kv = 0;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *conv_w = nullptr;
    DevWeight in_proj, out_proj, q, k, v, o, gate, up, down;
    // int8 copies for the tensor-core prefill GEMM (gemm_tc.cu); q == nullptr when unavailable
    TcWeight tc_in_proj, tc_out_proj, tc_q, tc_k, tc_v, tc_o, tc_gate, tc_up, tc_down;
    float *k_cache = nullptr, *v_cache = nullptr;  // [max_seq][kv_dim]
    float* conv_state = nullptr;                   // [d_conv][hidden]
};

}  // namespace

struct wick_cuda_weight {
    DevWeight w;
    int device = 0;
    TcWeight tc;                // filled by the first wick_cuda_gemm_q8_tc call
    uint32_t* tc_err = nullptr;
};

struct wick_cuda_model {
    int device = 0;
    cudaStream_t stream = nullptr;
    wick_cuda_config cfg{};
    int head_dim = 0;
    std::vector<Layer> layers;
    DevWeight embd;
    TcWeight tc_embd;       // tensor-core copy of the vocabulary matrix, made for the multi-sequence step only
    bool embd_q6k = false;  // token_embd is Q6_K: embd6 is used for the embedding rows and the logits, embd is empty
    DevQ6K embd6;
    float* output_norm = nullptr;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    int max_chunk = 0;  // tokens of scratch
    // tensor-core prefill GEMMs: available when every matrix meets tc_gemm_supported(); prefill_mode
    // picks the bit-exact one (default), the fused-chain one, or the bit-exact CUDA-core kernel
    bool tc_ok = false;     // the model's shapes allow the tensor-core GEMM
    bool tc_built = false;  // its int8 weight copies and buffers exist (made by the first call that needs them)
    int prefill_mode = WICK_CUDA_PREFILL_EXACT;
    CUtensorMap map_x_hs[2], map_x_is[2];  // activations [max_chunk][hs | is], box of 64 / 128 rows
    int8_t* q8m = nullptr;                  // lane-group-masked activations [4 * max_chunk][hs | is] (exact tensor-core GEMM)
    CUtensorMap map_xm_hs, map_xm_is, map_xm_hs32, map_xm_is32;  // boxes of 64 rows (16 tokens) and of 32 rows (8 tokens)
    float* normed_last = nullptr;  // output-normed hidden row of the last prefilled token
    float* rope_delta = nullptr;   // [head_dim]: cos then sin of the n_keep shift rotation
    uint32_t* tc_err = nullptr;
    // scratch, token-major
    float *hidden = nullptr, *block_out = nullptr, *ffn_out = nullptr, *proj = nullptr, *qbuf = nullptr, *kbuf = nullptr,
          *vbuf = nullptr, *attn_out = nullptr, *gate = nullptr, *up = nullptr, *logits = nullptr;
    float* q8s = nullptr;
    int8_t* q8q = nullptr;
    uint32_t* tokens_dev = nullptr;
    DecodeCtl* ctl = nullptr;
    uint32_t* argmax_tok = nullptr;
    uint32_t* ring = nullptr;
    int ring_len = 0;
    // pinned host staging
    uint32_t* h_u32 = nullptr;   // [ring_len] tokens in / out
    float* h_logits = nullptr;   // [vocab]
    cudaGraphExec_t g_logits = nullptr, g_greedy = nullptr;
    uint64_t nodes_logits = 0, nodes_greedy = 0;  // kernels per graph replay
    uint64_t launches = 0;                        // kernels launched so far
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;     // bracket the GPU work of the last call
    // persistent decode kernel (decode_mega.cu); falls back to the captured graphs when the
    // model does not meet its layout requirements or WICK_CUDA_DECODE=graph is set
    bool mega_ok = false;
    int mega_ctas = 0;
    MegaParams mega{};
    MegaPhase* d_phases = nullptr;
    MegaPhase* d_phases_long = nullptr;  // the same list with an MPH_SCORES phase before every MPH_ATTN (long contexts)
    int n_phases_long = 0;
    float* scores_g = nullptr;
    bool last_launch_long = false, long_ok = false;
    MegaLayer* d_mlayers = nullptr;
    unsigned long long* d_sync = nullptr;  // [0] barrier counter, [1..2] argmax accumulators
    unsigned long long* hidden_flagged = nullptr;  // [hs] flagged copy of the hidden row (persistent decode kernel)
    unsigned long long* d_prof = nullptr;  // [n_phases][4] timestamps of the last step
    unsigned long long bar_base = 0;
    DecodeCtl* h_ctl = nullptr;            // pinned copy of the control block
    uint32_t seq_len = 0;
    uint64_t bytes = 0;
    std::vector<void*> allocs;
    // extra sequence slots for wick_cuda_decode_batch (the model's own sequence is not one of them)
    struct SeqSlot {
        bool live = false;
        uint32_t seq_len = 0;
        std::vector<float*> k_cache, v_cache, conv_state;  // per layer (NULL where the layer has none)
    };
    std::vector<SeqSlot> seqs;
    // per-category device timers of the prefill pipeline (WICK_CUDA_PROFILE=events or wick_cuda_profile_enable)
    bool prof_on = false;
    std::vector<cudaEvent_t> prof_events;   // pool, reused chunk after chunk
    std::vector<int> prof_marks;            // category that ENDS at event i + 1 of the current chunk
    size_t prof_used = 0;
    double prof_ms[WICK_CUDA_PROFILE_CATEGORIES] = {};
    // opt-in split-K decode attention (graph decode path and the multi-sequence step; the persistent kernel stays exact)
    bool attn_splitk = false;
    float* splitk_scratch = nullptr;
    size_t splitk_floats = 0;
    float* sample_val = nullptr;        // [vocab] work arrays of the on-device sampler, made on first use
    int* sample_idx = nullptr;
    uint32_t* sample_status = nullptr;
    int batch_cap = 0;                  // rows the batch buffers below hold
    float* logits_rows = nullptr;       // [batch_cap][vocab]
    uint32_t *rows_tok = nullptr, *rows_next = nullptr, *rows_pos = nullptr, *rows_out = nullptr;  // device; rows_out [steps][rows]
    size_t rows_out_cap = 0;
    float** rows_ptrs = nullptr;        // device [n_layers][2][batch_cap] per-row state pointers
    uint8_t* h_rows = nullptr;          // pinned staging for tokens, positions, pointers and results
    size_t h_rows_bytes = 0;

    ~wick_cuda_model() {
        cudaSetDevice(device);
        if (stream) cudaStreamSynchronize(stream);
        if (g_logits) cudaGraphExecDestroy(g_logits);
        if (g_greedy) cudaGraphExecDestroy(g_greedy);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
        for (cudaEvent_t e : prof_events) cudaEventDestroy(e);
        for (void* p : allocs) cudaFree(p);
        if (h_u32) cudaFreeHost(h_u32);
        if (h_logits) cudaFreeHost(h_logits);
        if (h_ctl) cudaFreeHost(h_ctl);
        if (h_rows) cudaFreeHost(h_rows);
        if (stream) cudaStreamDestroy(stream);
    }
};

namespace {

template <class T>
int32_t dev_alloc(wick_cuda_model* m, T** out, size_t count) {
    void* p = nullptr;
    size_t bytes = std::max<size_t>(count * sizeof(T), 256);
    CU_TRY(cudaMalloc(&p, bytes));
    m->allocs.push_back(p);
    m->bytes += bytes;
    *out = (T*)p;
    return WICK_CUDA_OK;
}

int32_t upload_f32(wick_cuda_model* m, const GgufImage& g, const std::string& name, size_t expect, float** out) {
    const GgufTensor* t = g.tensor(name);
    if (!t) return fail(WICK_CUDA_ERR_BAD_GGUF, "tensor not found: " + name);
    uint64_t ne = 1;
    for (uint64_t d : t->dims) ne *= d;
    if (ne != expect) return fail(WICK_CUDA_ERR_BAD_GGUF, "tensor " + name + ": unexpected element count");
    std::vector<float> host(ne);
    if (t->type == 0) {
        memcpy(host.data(), g.data() + t->offset, ne * 4);
    } else if (t->type == 1) {
        const __half* h = (const __half*)(g.data() + t->offset);
        for (uint64_t i = 0; i < ne; i++) host[i] = __half2float(h[i]);
    } else {
        return fail(WICK_CUDA_ERR_UNSUPPORTED_DTYPE, "tensor " + name + ": expected F32 or F16");
    }
    W_TRY(dev_alloc(m, out, ne));
    CU_TRY(cudaMemcpy(*out, host.data(), ne * 4, cudaMemcpyHostToDevice));
    return WICK_CUDA_OK;
}

// Uploads GGUF block rows and re-lays them out into planes (see DevWeight).
int32_t upload_weight_raw(const DevWeight& w, const uint8_t* raw_host, uint8_t* staging, cudaStream_t st, uint8_t* q_dev,
                          __half* d_dev) {
    size_t nblk = (size_t)w.m * (w.k / QK);
    size_t raw_bytes = nblk * (w.dtype == DT_Q4_0 ? 18 : 34);
    CU_TRY(cudaMemcpyAsync(staging, raw_host, raw_bytes, cudaMemcpyHostToDevice, st));
    launch_repack(st, w, staging, q_dev, d_dev);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(st));
    return WICK_CUDA_OK;
}

int32_t upload_weight(wick_cuda_model* m, const GgufImage& g, const std::string& name, int expect_m, int expect_k,
                      uint8_t* staging, DevWeight* out) {
    const GgufTensor* t = g.tensor(name);
    if (!t) return fail(WICK_CUDA_ERR_BAD_GGUF, "tensor not found: " + name);
    if (t->type != DT_Q4_0 && t->type != DT_Q8_0)
        return fail(WICK_CUDA_ERR_UNSUPPORTED_DTYPE,
                    "tensor " + name + ": ggml type " + std::to_string(t->type) + " (only Q4_0 and Q8_0 are supported)");
    // GGUF shape [inner, outer] -> rows of `inner` elements (lfm2.rs:323-329)
    int k = t->dims.size() > 0 ? (int)t->dims[0] : 1;
    int rows = t->dims.size() > 1 ? (int)t->dims[1] : 1;
    if (rows != expect_m || k != expect_k || k % QK)
        return fail(WICK_CUDA_ERR_BAD_GGUF, "tensor " + name + ": shape [" + std::to_string(k) + "," + std::to_string(rows) +
                                                "] does not match the model config");
    DevWeight w;
    w.m = rows;
    w.k = k;
    w.dtype = (int)t->type;
    uint8_t* q = nullptr;
    __half* d = nullptr;
    W_TRY(dev_alloc(m, &q, w.q_bytes()));
    W_TRY(dev_alloc(m, &d, w.d_bytes() / 2));
    W_TRY(upload_weight_raw(w, g.data() + t->offset, staging, m->stream, q, d));
    w.q = q;
    w.d = d;
    *out = w;
    return WICK_CUDA_OK;
}

// token_embd in Q6_K: raw super-blocks to the device, then split into the planes of DevQ6K.
int32_t upload_q6k(wick_cuda_model* m, const GgufImage& g, const std::string& name, int expect_m, int expect_k, uint8_t* staging,
                   DevQ6K* out) {
    const GgufTensor* t = g.tensor(name);
    if (!t) return fail(WICK_CUDA_ERR_BAD_GGUF, "tensor not found: " + name);
    int k = t->dims.size() > 0 ? (int)t->dims[0] : 1;
    int rows = t->dims.size() > 1 ? (int)t->dims[1] : 1;
    if (rows != expect_m || k != expect_k || k % QK_K)
        return fail(WICK_CUDA_ERR_BAD_GGUF, "tensor " + name + ": Q6_K shape [" + std::to_string(k) + "," + std::to_string(rows) +
                                                "] does not match the model config (row length must be a multiple of 256)");
    if (gemv_q6k_smem(k) > 48 * 1024) return fail(WICK_CUDA_ERR_UNSUPPORTED_DTYPE, "Q6_K rows longer than 6144 elements are not supported");
    DevQ6K w;
    w.m = rows;
    w.k = k;
    uint8_t *ql = nullptr, *qh = nullptr;
    int8_t* sc = nullptr;
    __half* d = nullptr;
    W_TRY(dev_alloc(m, &ql, (size_t)rows * (k / 2)));
    W_TRY(dev_alloc(m, &qh, (size_t)rows * (k / 4)));
    W_TRY(dev_alloc(m, &sc, (size_t)rows * (k / 16)));
    W_TRY(dev_alloc(m, &d, (size_t)rows * (k / QK_K)));
    w.ql = ql; w.qh = qh; w.sc = sc; w.d = d;
    const size_t raw_bytes = (size_t)rows * (k / QK_K) * 210;
    CU_TRY(cudaMemcpyAsync(staging, g.data() + t->offset, raw_bytes, cudaMemcpyHostToDevice, m->stream));
    launch_repack_q6k(m->stream, staging, w);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(m->stream));
    *out = w;
    return WICK_CUDA_OK;
}

// cos / sin of every (position, pair) evaluated with the host libm in the reference's order
// (cpu.rs:2145-2158): theta starts at pos as f32 and is multiplied by powf(base, -2/hd).
void fill_rope_table(int n_pos, int hd, float base, std::vector<float>& c, std::vector<float>& s) {
    int half = hd / 2;
    c.resize((size_t)n_pos * half);
    s.resize((size_t)n_pos * half);
    float theta_scale = powf(base, -2.0f / (float)hd);
    for (int p = 0; p < n_pos; p++) {
        float theta = (float)p;
        for (int i = 0; i < half; i++) {
            c[(size_t)p * half + i] = cosf(theta);
            s[(size_t)p * half + i] = sinf(theta);
            theta *= theta_scale;
        }
    }
}

// Phase list of one decode step for the persistent kernel (see decode_mega.cu).
int32_t build_mega(wick_cuda_model* m) {
    const char* env = getenv("WICK_CUDA_DECODE");
    if (env && std::string(env) == "graph") return WICK_CUDA_OK;
    int coop = 0;
    CU_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, m->device));
    if (!coop) return WICK_CUDA_OK;
    const wick_cuda_config& c = m->cfg;
    const int hs = c.hidden_size, is = c.intermediate_size;
    std::vector<MegaPhase> ph;
    std::vector<MegaLayer> ml(c.n_layers);
    size_t max_group = 0;
    bool ok = true;
    auto mat = [&](const DevWeight& w, float* y, int epi) {
        MegaMat mm{};
        mm.w = w;
        mm.y = y;
        mm.epi = epi;
        if (w.k % 64) ok = false;  // an even block count keeps every bulk copy 16-byte sized
        max_group = std::max(max_group, w.q_group_bytes() + w.d_group_bytes());
        return mm;
    };
    int pending_commit = -1;
    for (uint32_t i = 0; i < c.n_layers; i++) {
        Layer& L = m->layers[i];
        MegaLayer& M = ml[i];
        M.conv_w = L.conv_w; M.conv_state = L.conv_state; M.q_norm = L.q_norm; M.k_norm = L.k_norm;
        M.k_cache = L.k_cache; M.v_cache = L.v_cache; M.n_kv = L.n_kv;
        MegaPhase a{};
        a.kind = MPH_NORM; a.k = hs; a.layer = (int)i; a.embed = i == 0; a.conv_commit = -1; a.norm_w = L.attn_norm;
        if (!L.is_attn) {
            a.n_mat = 1; a.mat[0] = mat(L.in_proj, m->proj, MEP_STORE);
            ph.push_back(a);
            MegaPhase b{};
            b.kind = MPH_CONV; b.k = hs; b.layer = (int)i; b.conv_commit = -1; b.n_mat = 1;
            b.mat[0] = mat(L.out_proj, m->hidden, MEP_ADD);
            ph.push_back(b);
            pending_commit = (int)i;
        } else {
            a.n_mat = 3;
            a.mat[0] = mat(L.q, m->qbuf, MEP_STORE);
            a.mat[1] = mat(L.k, m->kbuf, MEP_STORE);
            a.mat[2] = mat(L.v, m->vbuf, MEP_STORE);
            ph.push_back(a);
            MegaPhase at{};
            at.kind = MPH_ATTN; at.layer = (int)i; at.conv_commit = -1; at.k = hs;
            ph.push_back(at);
            MegaPhase o{};
            o.kind = MPH_QUANT; o.src = m->attn_out; o.k = hs; o.layer = (int)i; o.conv_commit = -1; o.n_mat = 1;
            o.mat[0] = mat(L.o, m->hidden, MEP_ADD);
            ph.push_back(o);
        }
        MegaPhase f{};
        f.kind = MPH_NORM; f.k = hs; f.layer = (int)i; f.conv_commit = pending_commit; f.norm_w = L.ffn_norm; f.n_mat = 2;
        pending_commit = -1;
        // gate and up of equal shape and type are streamed as alternating stages and SwiGLU is applied
        // by the thread that holds both sums of a row; `gate` then holds silu(gate) * up
        const bool fuse = L.gate.m == L.up.m && L.gate.k == L.up.k && L.gate.dtype == L.up.dtype;
        f.pair = fuse ? 1 : 0;
        f.mat[0] = mat(L.gate, m->gate, fuse ? MEP_SWIGLU : MEP_STORE);
        f.mat[1] = mat(L.up, m->up, fuse ? MEP_SWIGLU : MEP_STORE);
        ph.push_back(f);
        MegaPhase d{};
        d.kind = fuse ? MPH_QUANT : MPH_SILU; d.src = m->gate; d.k = is; d.layer = (int)i; d.conv_commit = -1; d.n_mat = 1;
        d.mat[0] = mat(L.down, m->hidden, MEP_ADD);
        ph.push_back(d);
    }
    if (!m->embd_q6k) {
        MegaPhase v{};
        v.kind = MPH_NORM; v.k = hs; v.layer = -1; v.conv_commit = -1; v.norm_w = m->output_norm; v.n_mat = 1;
        v.mat[0] = mat(m->embd, m->logits, MEP_LOGITS);
        ph.push_back(v);
    }  // a Q6_K vocabulary matrix is not streamed by the persistent kernel: see run_mega
    if (!ok || c.conv_kernel_size < 2 || c.conv_kernel_size > 4 || m->head_dim > 256 || m->head_dim % 16 || std::max(hs, is) > MEGA_CONSUMER_WARPS * 16 * 32) return WICK_CUDA_OK;

    MegaParams& P = m->mega;
    P.n_phases = (int)ph.size();
    P.n_layers = (int)ml.size();
    P.hs = hs; P.is = is; P.n_heads = c.n_heads; P.head_dim = m->head_dim; P.vocab = c.vocab_size;
    P.conv_ks = c.conv_kernel_size; P.max_seq = c.max_seq_len; P.eps = c.rms_norm_eps;
    P.embd = m->embd;
    P.embd_q6k = m->embd_q6k ? 1 : 0;
    P.skip_logits = m->embd_q6k ? 1 : 0;
    P.embd6 = m->embd6;
    P.hidden = m->hidden; P.proj = m->proj; P.qbuf = m->qbuf; P.kbuf = m->kbuf; P.vbuf = m->vbuf;
    P.attn_out = m->attn_out; P.gate = m->gate; P.up = m->up; P.logits = m->logits;
    P.rope_cos = m->rope_cos; P.rope_sin = m->rope_sin;
    P.ctl = m->ctl; P.ring = m->ring; P.ring_len = m->ring_len;
    P.kmax = std::max(hs, is);
    P.slot_bytes = (int)std::max<size_t>(16384, (max_group + 1023) / 1024 * 1024);
    P.n_slots = 0;
    P.xf_extra = 0;
    P.uniform_dtype = 0;
    {
        int dt = -1;
        bool same = true;
        for (const MegaPhase& q : ph)
            for (int i = 0; i < q.n_mat; i++) {
                if (dt < 0) dt = q.mat[i].w.dtype;
                same = same && q.mat[i].w.dtype == dt;
            }
        if (same && (dt == DT_Q4_0 || dt == DT_Q8_0)) P.uniform_dtype = dt;
    }
    int max_smem = 0;
    CU_TRY(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, m->device));
    const int n_phases_short = P.n_phases;
    P.n_phases = (int)ph.size() + (int)std::count_if(ph.begin(), ph.end(), [](const MegaPhase& q) { return q.kind == MPH_ATTN; });
    size_t fixed = mega_smem_bytes(P);  // sized for the longer of the two phase lists
    if (fixed + MEGA_TEAMS * ((size_t)P.slot_bytes + 16) + 64 * 4 > (size_t)max_smem) return WICK_CUDA_OK;
    P.n_slots = (int)(((size_t)max_smem - fixed - 64 * 4) / ((size_t)P.slot_bytes + 16));
    if (P.n_slots > 30) P.n_slots = 30;
    P.n_slots -= P.n_slots % MEGA_TEAMS;  // each slot is always served by the same consumer team
    if (P.n_slots % (2 * MEGA_TEAMS))       // paired (gate/up) phases need whole pairs per ring lap
        for (auto& q : ph) if (q.pair) { q.pair = 0; q.mat[0].epi = q.mat[1].epi = MEP_STORE; }
    for (size_t i = 0; i + 1 < ph.size(); i++)
        if (ph[i].kind == MPH_NORM && ph[i].n_mat == 2 && !ph[i].pair && ph[i + 1].kind == MPH_QUANT && ph[i + 1].src == m->gate) ph[i + 1].kind = MPH_SILU;
    // A residual-add phase followed by an RMSNorm phase hands the hidden row over through flagged words instead of
    // a grid barrier (WICK_CUDA_NO_FLAGGED_HIDDEN keeps the barrier, for A/B measurements).
    if (hs <= MEGA_FLAGGED_MAX_K && getenv("WICK_CUDA_NO_FLAGGED_HIDDEN") == nullptr)
        for (size_t i = 0; i + 1 < ph.size(); i++)
            if (ph[i].n_mat == 1 && ph[i].mat[0].epi == MEP_ADD && ph[i].mat[0].y == m->hidden && ph[i + 1].kind == MPH_NORM && !ph[i + 1].embed && ph[i + 1].k == hs)
                ph[i].flag_out = ph[i + 1].flag_in = 1;
    // long-context variant of the list: the cached keys' scores are computed by a phase of their own, spread over all CTAs
    std::vector<MegaPhase> ph_long;
    for (const MegaPhase& q : ph) {
        if (q.kind == MPH_ATTN) {
            MegaPhase sc = q;
            sc.kind = MPH_SCORES;
            ph_long.push_back(sc);
        }
        ph_long.push_back(q);
    }
    m->n_phases_long = (int)ph_long.size();
    W_TRY(dev_alloc(m, &m->d_phases_long, ph_long.size()));
    W_TRY(dev_alloc(m, &m->scores_g, (size_t)c.n_heads * c.max_seq_len));
    CU_TRY(cudaMemcpy(m->d_phases_long, ph_long.data(), ph_long.size() * sizeof(MegaPhase), cudaMemcpyHostToDevice));
    W_TRY(dev_alloc(m, &m->d_phases, ph.size()));
    W_TRY(dev_alloc(m, &m->d_mlayers, ml.size()));
    W_TRY(dev_alloc(m, &m->d_sync, 4));
    W_TRY(dev_alloc(m, &m->hidden_flagged, (size_t)hs));
    CU_TRY(cudaMemset(m->hidden_flagged, 0, (size_t)hs * 8));
    W_TRY(dev_alloc(m, &m->d_prof, ph_long.size() * 4 + 16));
    CU_TRY(cudaMemset(m->d_prof, 0, (ph_long.size() * 4 + 16) * 8));
    P.prof = m->d_prof;
    P.prof_phase = getenv("WICK_CUDA_PROF_PHASE") ? atoi(getenv("WICK_CUDA_PROF_PHASE")) : -1;
    CU_TRY(cudaMemcpy(m->d_phases, ph.data(), ph.size() * sizeof(MegaPhase), cudaMemcpyHostToDevice));
    CU_TRY(cudaMemcpy(m->d_mlayers, ml.data(), ml.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice));
    CU_TRY(cudaMemset(m->d_sync, 0, 32));
    P.phases = m->d_phases;
    P.layers = m->d_mlayers;
    P.bar_counter = m->d_sync;
    P.hidden_flagged = m->hidden_flagged;
    P.argmax_acc = m->d_sync + 1;
    {   // hand the shared memory the ring leaves unused to the attention staging area
        const size_t used = mega_smem_bytes(P);  // still with the long list's phase count
        if ((size_t)max_smem > used + 1024) P.xf_extra = (int)(((size_t)max_smem - used - 1024) / 4) & ~15;
    }
    P.n_phases = n_phases_short;
    P.long_ctx = 0;
    P.scores_g = m->scores_g;
    m->mega_ctas = mega_max_ctas(P);
    {   // the long-context instantiation must be co-resident on the same grid, or it is not used
        MegaParams PL = P;
        PL.long_ctx = 1;
        PL.n_phases = m->n_phases_long;
        PL.phases = m->d_phases_long;
        m->long_ok = mega_max_ctas(PL) >= m->mega_ctas;
    }
    m->mega_ok = m->mega_ctas > 0;
    return WICK_CUDA_OK;
}

// Runs n decode steps with the persistent kernel; ctl holds token / pos / step on entry.
void logits_matvec(wick_cuda_model* m);

// Contexts from this length on decode with the split-scores phase list (one extra grid barrier per attention layer,
// ~2.5 us, against a scores loop that grows by ~12 ns per cached key and CTA).
static const uint32_t MEGA_LONG_CTX = 768;

int32_t run_mega(wick_cuda_model* m, int n_tokens, bool greedy) {
    MegaParams P = m->mega;
    P.greedy = greedy ? 1 : 0;
    m->last_launch_long = m->long_ok && m->seq_len >= MEGA_LONG_CTX && getenv("WICK_CUDA_NO_SPLIT_SCORES") == nullptr;
    if (m->last_launch_long) {
        P.phases = m->d_phases_long;
        P.n_phases = m->n_phases_long;
        P.long_ctx = 1;
    }
    if (!P.skip_logits) {
        P.n_tokens = n_tokens;
        P.bar_base = m->bar_base;
        CU_TRY(launch_decode_mega(m->stream, P, m->mega_ctas));
        m->launches += 1;
        m->bar_base += (unsigned long long)n_tokens * P.n_phases;
    } else {
        // Q6_K vocabulary matrix: the persistent kernel runs the layers of ONE step; the output norm, the
        // Q6_K logits mat-vec, the argmax and the control-block update follow as kernels on the same stream
        // (token and position stay on the device, so the host does not wait between steps)
        const unsigned long long before = g_kernel_launches;
        P.n_tokens = 1;
        for (int t = 0; t < n_tokens; t++) {
            P.bar_base = m->bar_base;
            CU_TRY(launch_decode_mega(m->stream, P, m->mega_ctas));
            m->bar_base += (unsigned long long)P.n_phases;
            launch_add_rmsnorm_quant(m->stream, m->hidden, nullptr, m->output_norm, m->cfg.rms_norm_eps, 1, m->cfg.hidden_size, m->q8s,
                                     m->q8q, nullptr);
            logits_matvec(m);
            if (greedy) {
                launch_argmax(m->stream, m->logits, m->cfg.vocab_size, &m->ctl->argmax, m->argmax_tok);
                launch_decode_advance(m->stream, m->ctl, m->argmax_tok, m->ring, m->ring_len);
            } else {
                launch_decode_advance(m->stream, m->ctl, &m->ctl->token, nullptr, 0);  // keeps the token, pos += 1
            }
        }
        m->launches += g_kernel_launches - before;
        CU_TRY(cudaGetLastError());
    }
    CU_TRY(cudaMemcpyAsync(m->h_ctl, m->ctl, sizeof(DecodeCtl), cudaMemcpyDeviceToHost, m->stream));
    return WICK_CUDA_OK;
}

int32_t check_mega_status(wick_cuda_model* m) {
    if (m->h_ctl->error) {
        uint32_t e = m->h_ctl->error;
        // the barrier counter is no longer in step with bar_base: resynchronise and clear
        cudaMemsetAsync(m->d_sync, 0, 32, m->stream);
        cudaMemsetAsync(m->hidden_flagged, 0, (size_t)m->cfg.hidden_size * 8, m->stream);  // phase ids restart with bar_base
        cudaMemsetAsync(&m->ctl->error, 0, 4, m->stream);
        cudaStreamSynchronize(m->stream);
        m->bar_base = 0;
        return fail(WICK_CUDA_ERR_TIMEOUT, "decode kernel gave up waiting (flags " + std::to_string(e) +
                                               "); the sequence state is undefined, reset before reuse");
    }
    return WICK_CUDA_OK;
}

size_t naive_attn_smem(const wick_cuda_model* m) { return naive_attention_smem_bytes(m->head_dim, (int)m->cfg.max_seq_len); }

// One decode step on the stream; token and position come from m->ctl (run_layers,
// lfm2.rs:1020-1124, then the tied-embedding logits GEMV, lfm2.rs:2268-2288).
// Embedding rows into m->hidden and the tied-embedding logits from the quantised normed row in m->q8*
// (lfm2.rs:621-643, :2268-2288), for either storage type of token_embd.
void embed_rows(wick_cuda_model* m, const uint32_t* tokens_dev, const DecodeCtl* ctl, int n) {
    if (m->embd_q6k) launch_embed_q6k(m->stream, m->embd6, tokens_dev, ctl, m->hidden, n);
    else launch_embed(m->stream, m->embd, tokens_dev, ctl, m->hidden, n);
}

void logits_matvec(wick_cuda_model* m) {
    if (m->embd_q6k) {
        launch_gemv_q6k(m->stream, m->embd6, m->q8s, m->q8q, m->logits);
    } else {
        GemvJob lg{};
        lg.count = 1; lg.w[0] = m->embd; lg.y[0] = m->logits;
        launch_gemv(m->stream, lg, m->q8s, m->q8q);
    }
}

int32_t ensure_splitk_scratch(wick_cuda_model* m, int rows) {
    const size_t need = attention_splitk_scratch_floats(rows, (int)m->cfg.n_heads, m->head_dim, (int)m->cfg.max_seq_len);
    if (need > m->splitk_floats) {
        W_TRY(dev_alloc(m, &m->splitk_scratch, need));
        m->splitk_floats = need;
    }
    return WICK_CUDA_OK;
}

void enqueue_decode(wick_cuda_model* m, bool greedy) {
    cudaStream_t st = m->stream;
    const int hs = m->cfg.hidden_size, is = m->cfg.intermediate_size, hd = m->head_dim;
    embed_rows(m, nullptr, m->ctl, 1);
    const float* pending = nullptr;  // block output not yet added to the residual stream
    for (size_t li = 0; li < m->layers.size(); li++) {
        Layer& L = m->layers[li];
        launch_add_rmsnorm_quant(st, m->hidden, pending, L.attn_norm, m->cfg.rms_norm_eps, 1, hs, m->q8s, m->q8q, nullptr);
        if (!L.is_attn) {
            GemvJob j{};
            j.count = 1; j.w[0] = L.in_proj; j.y[0] = m->proj;
            launch_gemv(st, j, m->q8s, m->q8q);
            launch_shortconv(st, m->proj, L.conv_w, L.conv_state, 1, hs, m->cfg.conv_kernel_size, nullptr, m->q8s, m->q8q);
            GemvJob o{};
            o.count = 1; o.w[0] = L.out_proj; o.y[0] = m->block_out;
            launch_gemv(st, o, m->q8s, m->q8q);
        } else {
            GemvJob j{};
            j.count = 3;
            j.w[0] = L.q; j.y[0] = m->qbuf;
            j.w[1] = L.k; j.y[1] = m->kbuf;
            j.w[2] = L.v; j.y[2] = m->vbuf;
            launch_gemv(st, j, m->q8s, m->q8q);
            launch_qknorm_rope_kv(st, m->qbuf, m->kbuf, m->vbuf, L.q_norm, L.k_norm, m->cfg.rms_norm_eps, m->rope_cos,
                                  m->rope_sin, L.k_cache, L.v_cache, 1, -1, m->ctl, m->cfg.n_heads, L.n_kv, hd);
            if (m->attn_splitk)
                launch_attention_splitk(st, m->qbuf, nullptr, nullptr, L.k_cache, L.v_cache, &m->ctl->pos, m->attn_out, m->splitk_scratch, 1,
                                        m->cfg.n_heads, L.n_kv, hd, m->cfg.max_seq_len);
            else
                launch_attention_naive(st, m->qbuf, L.k_cache, L.v_cache, m->attn_out, 1, -1, m->ctl, m->cfg.n_heads, L.n_kv, hd,
                                       m->cfg.max_seq_len);
            launch_quant_rows(st, m->attn_out, 1, hs, m->q8s, m->q8q);
            GemvJob o{};
            o.count = 1; o.w[0] = L.o; o.y[0] = m->block_out;
            launch_gemv(st, o, m->q8s, m->q8q);
        }
        launch_add_rmsnorm_quant(st, m->hidden, m->block_out, L.ffn_norm, m->cfg.rms_norm_eps, 1, hs, m->q8s, m->q8q, nullptr);
        GemvJob gu{};
        gu.count = 2;
        gu.w[0] = L.gate; gu.y[0] = m->gate;
        gu.w[1] = L.up; gu.y[1] = m->up;
        launch_gemv(st, gu, m->q8s, m->q8q);
        launch_silu_mul_quant(st, m->gate, m->up, 1, is, m->q8s, m->q8q, nullptr);
        GemvJob dn{};
        dn.count = 1; dn.w[0] = L.down; dn.y[0] = m->ffn_out;
        launch_gemv(st, dn, m->q8s, m->q8q);
        pending = m->ffn_out;
    }
    launch_add_rmsnorm_quant(st, m->hidden, pending, m->output_norm, m->cfg.rms_norm_eps, 1, hs, m->q8s, m->q8q, nullptr);
    logits_matvec(m);
    if (greedy) {
        launch_argmax(st, m->logits, m->cfg.vocab_size, &m->ctl->argmax, m->argmax_tok);
        launch_decode_advance(st, m->ctl, m->argmax_tok, m->ring, m->ring_len);
    } else {
        launch_decode_advance(st, m->ctl, &m->ctl->token, nullptr, 0);  // keeps the token, pos += 1
    }
}

int32_t capture_graph(wick_cuda_model* m, bool greedy, cudaGraphExec_t* out, uint64_t* nodes) {
    cudaGraph_t graph = nullptr;
    CU_TRY(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    const unsigned long long before = g_kernel_launches;
    enqueue_decode(m, greedy);
    *nodes = g_kernel_launches - before;
    cudaError_t e = cudaStreamEndCapture(m->stream, &graph);
    if (e != cudaSuccess) return fail(WICK_CUDA_ERR_CUDA, std::string("graph capture: ") + cudaGetErrorString(e));
    e = cudaGraphInstantiate(out, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail(WICK_CUDA_ERR_CUDA, std::string("graph instantiate: ") + cudaGetErrorString(e));
    return WICK_CUDA_OK;
}

// Per-category device timers (the counterpart of wick's WICK_PROFILE=timing|gpu switches, metal_lfm2.rs:529-533,
// :596-600): an event after every group of kernels of one kind; the differences are added up per category once the
// chunk has finished.  Off by default: an event per kernel group costs a little launch time.
enum ProfCat { PC_EMBED = 0, PC_NORM_QUANT, PC_GEMM, PC_SHORTCONV, PC_QK_ROPE_KV, PC_ATTENTION, PC_ACT_QUANT, PC_LOGITS };
static const char* const PROF_NAMES[WICK_CUDA_PROFILE_CATEGORIES] = {"embedding", "rmsnorm+quantise", "gemm", "short-conv", "qk-norm+rope+kv-append",
                                                                      "attention", "activation+quantise", "output-norm+logits"};
void prof_begin(wick_cuda_model* m) {
    if (!m->prof_on) return;
    m->prof_used = 0;
    m->prof_marks.clear();
    if (m->prof_events.empty()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) == cudaSuccess) m->prof_events.push_back(e);
    }
    if (!m->prof_events.empty()) {
        cudaEventRecord(m->prof_events[0], m->stream);
        m->prof_used = 1;
    }
}
void prof_mark(wick_cuda_model* m, int cat) {  // the kernels enqueued since the previous mark belong to `cat`
    if (!m->prof_on || m->prof_used == 0) return;
    if (m->prof_used == m->prof_events.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return;
        m->prof_events.push_back(e);
    }
    cudaEventRecord(m->prof_events[m->prof_used++], m->stream);
    m->prof_marks.push_back(cat);
}
void prof_collect(wick_cuda_model* m) {  // after the stream has been synchronised
    if (!m->prof_on) return;
    for (size_t i = 0; i + 1 < m->prof_used; i++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, m->prof_events[i], m->prof_events[i + 1]) == cudaSuccess) m->prof_ms[m->prof_marks[i]] += ms;
    }
    m->prof_used = 0;
}

// Integer GEMMs of n quantised rows (m->q8q / m->q8s) with up to three matrices that read the same input, as one
// launch on the tensor cores when the chunk is wide enough to fill an MMA tile, else the exact CUDA-core kernel.
struct GemmTarget {
    const DevWeight* w;
    const TcWeight* t;
    float* out;
};
void run_gemms(wick_cuda_model* m, int n, std::initializer_list<GemmTarget> list) {
    cudaStream_t st = m->stream;
    const int hs = m->cfg.hidden_size;
    const bool tc = m->tc_built && n >= 16 && m->prefill_mode != WICK_CUDA_PREFILL_EXACT_CUDA_CORES;
    const bool tc_exact = tc && m->prefill_mode == WICK_CUDA_PREFILL_EXACT;
    if (tc) {
        const TcWeight* tw[3];
        float* outs[3];
        int c = 0;
        for (const GemmTarget& g : list) {
            tw[c] = g.t;
            outs[c++] = g.out;
        }
        const bool is_hs = tw[0]->k == hs;
        cudaError_t e;
        if (tc_exact) {
            launch_tc_mask_expand(st, m->q8q, n, tw[0]->k, m->q8m);
            e = launch_gemm_tc_exact(st, tw, outs, c, is_hs ? m->map_xm_hs : m->map_xm_is, m->q8s, n, m->tc_err,
                                     is_hs ? &m->map_xm_hs32 : &m->map_xm_is32);
        } else {
            e = launch_gemm_tc(st, tw, outs, c, is_hs ? m->map_x_hs : m->map_x_is, m->q8s, n, nullptr, m->tc_err);
        }
        (void)e;  // surfaced by the cudaGetLastError() check after the chunk
    } else {
        for (const GemmTarget& g : list) launch_gemm(st, *g.w, m->q8s, m->q8q, n, g.out);
    }
}

// One internal prefill chunk of n <= max_chunk tokens already in m->tokens_dev
// (prefill_layers_and_logits, lfm2.rs:1139-2213, aarch64 non-BLAS branch).
// `embed`: fill hidden from the token ids (false: the caller has copied input embeddings into m->hidden).
// `last`: this chunk ends the call: the last row goes through the output norm and then, with `want_logits`,
// through the vocabulary head (always leaving the normed row in m->normed_last).
void enqueue_prefill_chunk(wick_cuda_model* m, int n, int start_pos, bool flash, bool last, bool embed = true,
                           bool want_logits = true) {
    cudaStream_t st = m->stream;
    const int hs = m->cfg.hidden_size, is = m->cfg.intermediate_size, hd = m->head_dim;
    const float eps = m->cfg.rms_norm_eps;
    auto gemms = [&](std::initializer_list<GemmTarget> list) { run_gemms(m, n, list); };
    prof_begin(m);
    if (embed) embed_rows(m, m->tokens_dev, nullptr, n);
    prof_mark(m, PC_EMBED);
    const float* pending = nullptr;
    for (size_t li = 0; li < m->layers.size(); li++) {
        Layer& L = m->layers[li];
        launch_add_rmsnorm_quant(st, m->hidden, pending, L.attn_norm, eps, n, hs, m->q8s, m->q8q, nullptr);
        prof_mark(m, PC_NORM_QUANT);
        if (!L.is_attn) {
            gemms({{&L.in_proj, &L.tc_in_proj, m->proj}});
            prof_mark(m, PC_GEMM);
            launch_shortconv(st, m->proj, L.conv_w, L.conv_state, n, hs, m->cfg.conv_kernel_size, nullptr, m->q8s, m->q8q);
            prof_mark(m, PC_SHORTCONV);
            gemms({{&L.out_proj, &L.tc_out_proj, m->block_out}});
            prof_mark(m, PC_GEMM);
        } else {
            gemms({{&L.q, &L.tc_q, m->qbuf}, {&L.k, &L.tc_k, m->kbuf}, {&L.v, &L.tc_v, m->vbuf}});
            prof_mark(m, PC_GEMM);
            launch_qknorm_rope_kv(st, m->qbuf, m->kbuf, m->vbuf, L.q_norm, L.k_norm, eps, m->rope_cos, m->rope_sin, L.k_cache,
                                  L.v_cache, n, start_pos, nullptr, m->cfg.n_heads, L.n_kv, hd);
            prof_mark(m, PC_QK_ROPE_KV);
            if (flash)  // (shapes the tiled kernel does not take were refused when the model was created)
                launch_attention_flash(st, m->qbuf, L.k_cache, L.v_cache, m->attn_out, n, start_pos, m->cfg.n_heads, L.n_kv, hd, m->tc_err);
            else
                launch_attention_naive(st, m->qbuf, L.k_cache, L.v_cache, m->attn_out, n, start_pos, nullptr, m->cfg.n_heads,
                                       L.n_kv, hd, m->cfg.max_seq_len);
            prof_mark(m, PC_ATTENTION);
            launch_quant_rows(st, m->attn_out, n, hs, m->q8s, m->q8q);
            prof_mark(m, PC_ACT_QUANT);
            gemms({{&L.o, &L.tc_o, m->block_out}});
            prof_mark(m, PC_GEMM);
        }
        launch_add_rmsnorm_quant(st, m->hidden, m->block_out, L.ffn_norm, eps, n, hs, m->q8s, m->q8q, nullptr);
        prof_mark(m, PC_NORM_QUANT);
        gemms({{&L.gate, &L.tc_gate, m->gate}, {&L.up, &L.tc_up, m->up}});
        prof_mark(m, PC_GEMM);
        launch_silu_mul_quant(st, m->gate, m->up, n, is, m->q8s, m->q8q, nullptr);
        prof_mark(m, PC_ACT_QUANT);
        gemms({{&L.down, &L.tc_down, m->ffn_out}});
        prof_mark(m, PC_GEMM);
        pending = m->ffn_out;
    }
    if (last) {
        // last token only (lfm2.rs:2190-2212)
        size_t lastrow = (size_t)(n - 1) * hs;
        launch_add_rmsnorm_quant(st, m->hidden + lastrow, pending + lastrow, m->output_norm, eps, 1, hs, m->q8s, m->q8q, m->normed_last);
        if (want_logits) logits_matvec(m);
        prof_mark(m, PC_LOGITS);
    }
}

// Tensor-core prefill GEMM: decided at load (tc_ok = the shapes allow it), built on first use (ensure_tc): the int8
// copies of the layer matrices, the activation tensor maps and the masked-activation buffer cost about 1.7 bytes per
// parameter, which a decode-only user never needs.
int32_t build_tc(wick_cuda_model* m) {
    const int hs = m->cfg.hidden_size, is = m->cfg.intermediate_size;
    const char* mode = getenv("WICK_CUDA_PREFILL");
    m->prefill_mode = WICK_CUDA_PREFILL_EXACT;
    if (mode && strcmp(mode, "tensor") == 0) m->prefill_mode = WICK_CUDA_PREFILL_TENSOR;
    if (mode && strcmp(mode, "exact-cuda-cores") == 0) m->prefill_mode = WICK_CUDA_PREFILL_EXACT_CUDA_CORES;
    m->tc_ok = tc_gemm_supported(hs, hs) && tc_gemm_supported(hs, is);
    W_TRY(dev_alloc(m, &m->tc_err, 1));  // error word of the prefill kernels with bounded waits (GEMM and tiled attention)
    CU_TRY(cudaMemset(m->tc_err, 0, 4));
    if (!m->tc_ok && m->prefill_mode == WICK_CUDA_PREFILL_TENSOR) m->prefill_mode = WICK_CUDA_PREFILL_EXACT;
    return WICK_CUDA_OK;
}

int32_t ensure_tc(wick_cuda_model* m) {
    if (!m->tc_ok || m->tc_built || m->prefill_mode == WICK_CUDA_PREFILL_EXACT_CUDA_CORES) return WICK_CUDA_OK;
    const int hs = m->cfg.hidden_size, is = m->cfg.intermediate_size;
    auto fill = [&](const DevWeight& w, TcWeight* t) -> int32_t {
        t->m_pad = (w.m + 127) / 128 * 128;
        t->m = w.m;
        t->k = w.k;
        W_TRY(dev_alloc(m, &t->q, t->q_bytes()));
        W_TRY(dev_alloc(m, &t->scales_t, t->s_bytes() / sizeof(float)));
        CU_TRY(tc_weight_fill(m->stream, w, t));
        return WICK_CUDA_OK;
    };
    for (Layer& L : m->layers) {
        if (L.is_attn) {
            W_TRY(fill(L.q, &L.tc_q));
            W_TRY(fill(L.k, &L.tc_k));
            W_TRY(fill(L.v, &L.tc_v));
            W_TRY(fill(L.o, &L.tc_o));
        } else {
            W_TRY(fill(L.in_proj, &L.tc_in_proj));
            W_TRY(fill(L.out_proj, &L.tc_out_proj));
        }
        W_TRY(fill(L.gate, &L.tc_gate));
        W_TRY(fill(L.up, &L.tc_up));
        W_TRY(fill(L.down, &L.tc_down));
    }
    for (int i = 0; i < 2; i++) {
        CU_TRY(tc_make_activation_map(m->q8q, m->max_chunk, hs, i ? 128 : 64, &m->map_x_hs[i]));
        CU_TRY(tc_make_activation_map(m->q8q, m->max_chunk, is, i ? 128 : 64, &m->map_x_is[i]));
    }
    W_TRY(dev_alloc(m, &m->q8m, (size_t)4 * m->max_chunk * std::max(hs, is)));
    CU_TRY(tc_make_activation_map(m->q8m, 4 * m->max_chunk, hs, 64, &m->map_xm_hs));
    CU_TRY(tc_make_activation_map(m->q8m, 4 * m->max_chunk, is, 64, &m->map_xm_is));
    CU_TRY(tc_make_activation_map(m->q8m, 4 * m->max_chunk, hs, 32, &m->map_xm_hs32));
    CU_TRY(tc_make_activation_map(m->q8m, 4 * m->max_chunk, is, 32, &m->map_xm_is32));
    CU_TRY(cudaStreamSynchronize(m->stream));
    m->tc_built = true;
    return WICK_CUDA_OK;
}

int32_t reset_sequence(wick_cuda_model* m) {
    const int hs = m->cfg.hidden_size, dc = (int)m->cfg.conv_kernel_size - 1;
    for (Layer& L : m->layers)
        if (!L.is_attn && dc > 0) CU_TRY(cudaMemsetAsync(L.conv_state, 0, (size_t)dc * hs * sizeof(float), m->stream));
    DecodeCtl z{};
    // pinned staging keeps the copy asynchronous and ordered on the stream
    memcpy(m->h_u32, &z, sizeof(z));
    CU_TRY(cudaMemcpyAsync(m->ctl, m->h_u32, sizeof(z), cudaMemcpyHostToDevice, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    m->seq_len = 0;
    return WICK_CUDA_OK;
}

int32_t build_model(wick_cuda_model* m, const GgufImage& g, uint32_t context_size) {
    // config: Lfm2Model::from_gguf_with_id, lfm2.rs:97-185
    std::string arch;
    if (!g.get_str("general.architecture", &arch) || arch != "lfm2")
        return fail(WICK_CUDA_ERR_BAD_GGUF, "unsupported architecture: " + (arch.empty() ? std::string("unknown") : arch));
    if (context_size == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "context_size must be > 0");
    wick_cuda_config& c = m->cfg;
    if (!g.get_u32("lfm2.block_count", &c.n_layers)) return fail(WICK_CUDA_ERR_BAD_GGUF, "missing lfm2.block_count");
    if (!g.get_u32("lfm2.embedding_length", &c.hidden_size)) return fail(WICK_CUDA_ERR_BAD_GGUF, "missing lfm2.embedding_length");
    if (!g.get_u32("lfm2.feed_forward_length", &c.intermediate_size))
        return fail(WICK_CUDA_ERR_BAD_GGUF, "missing lfm2.feed_forward_length");
    if (!g.get_u32("lfm2.attention.head_count", &c.n_heads)) return fail(WICK_CUDA_ERR_BAD_GGUF, "missing lfm2.attention.head_count");
    if (!g.get_u32("lfm2.vocab_size", &c.vocab_size)) return fail(WICK_CUDA_ERR_BAD_GGUF, "missing lfm2.vocab_size");
    uint32_t gguf_ctx = 128000;
    g.get_u32("lfm2.context_length", &gguf_ctx);
    c.max_seq_len = std::min(context_size, gguf_ctx);
    c.rope_theta = 1000000.0f;
    g.get_f32("lfm2.rope.freq_base", &c.rope_theta);
    c.rms_norm_eps = 1e-5f;
    g.get_f32("lfm2.attention.layer_norm_rms_epsilon", &c.rms_norm_eps);
    c.conv_kernel_size = 3;
    g.get_u32("lfm2.shortconv.l_cache", &c.conv_kernel_size);
    std::vector<int32_t> kvh;
    if (!g.get_i32_array("lfm2.attention.head_count_kv", &kvh)) return fail(WICK_CUDA_ERR_BAD_GGUF, "missing lfm2.attention.head_count_kv");
    if (kvh.size() < c.n_layers)
        return fail(WICK_CUDA_ERR_BAD_GGUF, "head_count_kv array length (" + std::to_string(kvh.size()) + ") < block_count (" +
                                                std::to_string(c.n_layers) + ")");
    if (!c.n_layers || !c.hidden_size || !c.n_heads || c.hidden_size % c.n_heads || !c.vocab_size || !c.intermediate_size)
        return fail(WICK_CUDA_ERR_BAD_GGUF, "inconsistent model dimensions");
    const int hs = c.hidden_size, is = c.intermediate_size;
    m->head_dim = hs / c.n_heads;
    const int hd = m->head_dim;
    if (hs % QK || is % QK) return fail(WICK_CUDA_ERR_BAD_GGUF, "hidden and feed-forward sizes must be multiples of 32");
    if (hd % 8 || hd > 256) return fail(WICK_CUDA_ERR_BAD_GGUF, "head_dim must be a multiple of 8 and <= 256");
    if (c.conv_kernel_size < 1 || c.conv_kernel_size > 8) return fail(WICK_CUDA_ERR_BAD_GGUF, "unsupported shortconv.l_cache");
    if (naive_attn_smem(m) > 200 * 1024)
        return fail(WICK_CUDA_ERR_BAD_ARG, "context_size too large for the exact attention kernel (max ~51000 positions)");

    CU_TRY(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));

    size_t max_raw = 0;
    m->layers.resize(c.n_layers);
    c.n_kv_heads = 0;
    for (uint32_t i = 0; i < c.n_layers; i++) {
        Layer& L = m->layers[i];
        L.is_attn = g.tensor("blk." + std::to_string(i) + ".attn_q.weight") != nullptr;  // lfm2.rs:154
        if (L.is_attn) {
            int nkv = kvh[i];
            if (nkv <= 0 || c.n_heads % nkv)
                return fail(WICK_CUDA_ERR_BAD_GGUF, "layer " + std::to_string(i) + ": n_kv_heads (" + std::to_string(nkv) +
                                                        ") must be > 0 and divide n_heads (" + std::to_string(c.n_heads) + ")");
            L.n_kv = nkv;
            c.n_kv_heads = std::max<uint32_t>(c.n_kv_heads, nkv);
            // prompts of 256 tokens and more take the tiled attention kernel (lfm2.rs:1646-1647): refuse shapes it lacks
            if (!attention_flash_supported((int)c.n_heads, nkv, hd))
                return fail(WICK_CUDA_ERR_UNSUPPORTED_DTYPE, "layer " + std::to_string(i) + ": attention with head_dim " + std::to_string(hd) + " and " +
                                                                 std::to_string(c.n_heads / nkv) + " query heads per KV head is not supported "
                                                                 "(head_dim 32, 64 or 128; at most 8 query heads per KV head)");
        }
    }
    // staging buffer for the largest quantised tensor
    max_raw = (size_t)std::max<size_t>((size_t)c.vocab_size * hs, (size_t)3 * hs * std::max(hs, is)) / QK * 34;
    uint8_t* staging = nullptr;
    CU_TRY(cudaMalloc((void**)&staging, max_raw));
    struct StagingGuard {
        uint8_t* p;
        ~StagingGuard() { cudaFree(p); }
    } guard{staging};

    {
        const GgufTensor* te = g.tensor("token_embd.weight");
        if (te && te->type == DT_Q6_K) W_TRY(upload_q6k(m, g, "token_embd.weight", c.vocab_size, hs, staging, &m->embd6));
        else W_TRY(upload_weight(m, g, "token_embd.weight", c.vocab_size, hs, staging, &m->embd));
        m->embd_q6k = te && te->type == DT_Q6_K;
    }
    W_TRY(upload_f32(m, g, "token_embd_norm.weight", hs, &m->output_norm));  // the OUTPUT norm, lfm2.rs:188
    const int dc = (int)c.conv_kernel_size - 1;
    for (uint32_t i = 0; i < c.n_layers; i++) {
        Layer& L = m->layers[i];
        std::string p = "blk." + std::to_string(i) + ".";
        W_TRY(upload_f32(m, g, p + "attn_norm.weight", hs, &L.attn_norm));
        W_TRY(upload_f32(m, g, p + "ffn_norm.weight", hs, &L.ffn_norm));
        W_TRY(upload_weight(m, g, p + "ffn_gate.weight", is, hs, staging, &L.gate));
        W_TRY(upload_weight(m, g, p + "ffn_up.weight", is, hs, staging, &L.up));
        W_TRY(upload_weight(m, g, p + "ffn_down.weight", hs, is, staging, &L.down));
        if (L.is_attn) {
            int kv_dim = L.n_kv * hd;
            W_TRY(upload_weight(m, g, p + "attn_q.weight", hs, hs, staging, &L.q));
            W_TRY(upload_weight(m, g, p + "attn_k.weight", kv_dim, hs, staging, &L.k));
            W_TRY(upload_weight(m, g, p + "attn_v.weight", kv_dim, hs, staging, &L.v));
            W_TRY(upload_weight(m, g, p + "attn_output.weight", hs, hs, staging, &L.o));
            W_TRY(upload_f32(m, g, p + "attn_q_norm.weight", hd, &L.q_norm));
            W_TRY(upload_f32(m, g, p + "attn_k_norm.weight", hd, &L.k_norm));
            W_TRY(dev_alloc(m, &L.k_cache, (size_t)c.max_seq_len * kv_dim));
            W_TRY(dev_alloc(m, &L.v_cache, (size_t)c.max_seq_len * kv_dim));
        } else {
            W_TRY(upload_weight(m, g, p + "shortconv.in_proj.weight", 3 * hs, hs, staging, &L.in_proj));
            W_TRY(upload_weight(m, g, p + "shortconv.out_proj.weight", hs, hs, staging, &L.out_proj));
            W_TRY(upload_f32(m, g, p + "shortconv.conv.weight", (size_t)hs * c.conv_kernel_size, &L.conv_w));
            W_TRY(dev_alloc(m, &L.conv_state, (size_t)std::max(dc, 1) * hs));
        }
    }
    // RoPE table
    {
        std::vector<float> cs, sn;
        fill_rope_table(c.max_seq_len, hd, c.rope_theta, cs, sn);
        W_TRY(dev_alloc(m, &m->rope_cos, cs.size()));
        W_TRY(dev_alloc(m, &m->rope_sin, sn.size()));
        CU_TRY(cudaMemcpy(m->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
        CU_TRY(cudaMemcpy(m->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
    }
    // scratch
    // Tokens of activation scratch (longer prefill calls are cut into pieces of this size internally; results do not
    // depend on it).  The default is wick's own prefill chunk of 512 tokens (--ubatch-size); WICK_CUDA_MAX_CHUNK
    // overrides it (e.g. 4096: one GEMM pass per 4096-token call, at 0.45 GB more scratch for a 1.6B-class model).
    {
        int want = 512;
        if (const char* e = getenv("WICK_CUDA_MAX_CHUNK")) want = std::max(16, std::min(atoi(e), 8192));
        m->max_chunk = (int)std::min<uint32_t>(c.max_seq_len, (uint32_t)want);
    }
    const size_t N = m->max_chunk;
    const int kvmax = c.n_kv_heads * hd;
    W_TRY(dev_alloc(m, &m->hidden, N * hs));
    W_TRY(dev_alloc(m, &m->block_out, N * hs));
    W_TRY(dev_alloc(m, &m->ffn_out, N * hs));
    W_TRY(dev_alloc(m, &m->proj, N * 3 * hs));
    W_TRY(dev_alloc(m, &m->qbuf, N * hs));
    W_TRY(dev_alloc(m, &m->kbuf, N * std::max(kvmax, 1)));
    W_TRY(dev_alloc(m, &m->vbuf, N * std::max(kvmax, 1)));
    W_TRY(dev_alloc(m, &m->attn_out, N * hs));
    W_TRY(dev_alloc(m, &m->gate, N * is));
    W_TRY(dev_alloc(m, &m->up, N * is));
    W_TRY(dev_alloc(m, &m->logits, (size_t)c.vocab_size));
    W_TRY(dev_alloc(m, &m->q8s, N * (std::max(hs, is) / QK)));
    W_TRY(dev_alloc(m, &m->q8q, N * std::max(hs, is)));
    W_TRY(dev_alloc(m, &m->tokens_dev, N));
    W_TRY(dev_alloc(m, &m->normed_last, (size_t)hs));
    W_TRY(dev_alloc(m, &m->rope_delta, (size_t)hd));
    W_TRY(dev_alloc(m, &m->ctl, 1));
    W_TRY(dev_alloc(m, &m->argmax_tok, 1));
    m->ring_len = (int)c.max_seq_len;
    W_TRY(dev_alloc(m, &m->ring, (size_t)m->ring_len));
    CU_TRY(cudaMallocHost((void**)&m->h_u32, std::max<size_t>((size_t)std::max<int>(m->ring_len, m->max_chunk) * 4, 256)));
    CU_TRY(cudaMallocHost((void**)&m->h_logits, (size_t)c.vocab_size * 4));
    CU_TRY(cudaMallocHost((void**)&m->h_ctl, sizeof(DecodeCtl)));
    memset(m->h_ctl, 0, sizeof(DecodeCtl));
    CU_TRY(cudaMemset(m->ctl, 0, sizeof(DecodeCtl)));
    W_TRY(reset_sequence(m));
    if (naive_attn_smem(m) > 48 * 1024) {
        configure_naive_attention_smem(naive_attn_smem(m));
    }
    CU_TRY(cudaEventCreate(&m->ev0));
    CU_TRY(cudaEventCreate(&m->ev1));
    {
        const char* pe = getenv("WICK_CUDA_PROFILE");
        m->prof_on = pe && strcmp(pe, "events") == 0;
    }
    W_TRY(build_tc(m));
    W_TRY(build_mega(m));
    {
        const char* da = getenv("WICK_CUDA_DECODE_ATTENTION");
        if (da && strcmp(da, "splitk") == 0) {
            W_TRY(ensure_splitk_scratch(m, 1));
            m->attn_splitk = true;
        }
    }
    W_TRY(capture_graph(m, false, &m->g_logits, &m->nodes_logits));
    W_TRY(capture_graph(m, true, &m->g_greedy, &m->nodes_greedy));
    CU_TRY(cudaStreamSynchronize(m->stream));
    return WICK_CUDA_OK;
}

int32_t check_model(const wick_cuda_model* m) {
    if (!m) return fail(WICK_CUDA_ERR_BAD_ARG, "model handle is NULL");
    return WICK_CUDA_OK;
}

// ── sequence slots and the multi-sequence decode step ──────────────────────
// wick keeps one sequence per model (wick/src/model/mod.rs:56-71).  A slot is one more sequence's state (K / V caches,
// rolling conv buffers, length) on the same weights; wick_cuda_decode_batch advances many slots in one pass over the
// weights.  The model's own sequence (the one the Model-trait entry points use) is not a slot.
int32_t check_seq(const wick_cuda_model* m, uint32_t id) {
    if (id >= m->seqs.size() || !m->seqs[id].live) return fail(WICK_CUDA_ERR_BAD_ARG, "no such sequence slot: " + std::to_string(id));
    return WICK_CUDA_OK;
}

// Runs `fn` with the slot's state bound in place of the model's own sequence (the prefill drivers address the
// state through the layer table), then puts the model's own sequence back, device position included.
template <class F>
int32_t with_slot(wick_cuda_model* m, uint32_t id, F&& fn) {
    wick_cuda_model::SeqSlot& sl = m->seqs[id];
    auto swap_state = [&]() {
        for (size_t li = 0; li < m->layers.size(); li++) {
            Layer& L = m->layers[li];
            if (L.is_attn) {
                std::swap(L.k_cache, sl.k_cache[li]);
                std::swap(L.v_cache, sl.v_cache[li]);
            } else {
                std::swap(L.conv_state, sl.conv_state[li]);
            }
        }
        std::swap(m->seq_len, sl.seq_len);
    };
    swap_state();
    const int32_t r = fn();
    swap_state();
    m->h_u32[0] = m->seq_len;
    cudaError_t e = cudaMemcpyAsync(&m->ctl->pos, m->h_u32, 4, cudaMemcpyHostToDevice, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (r != WICK_CUDA_OK) return r;
    if (e != cudaSuccess) return fail(WICK_CUDA_ERR_CUDA, std::string("restoring the model's own sequence: ") + cudaGetErrorString(e));
    return WICK_CUDA_OK;
}

constexpr uint32_t MAX_BATCH_ROWS = 1024;

int32_t ensure_batch_buffers(wick_cuda_model* m, uint32_t rows, uint32_t steps) {
    const size_t nl = m->layers.size();
    if ((int)rows > m->batch_cap) {
        const int cap = (int)std::min<uint32_t>(std::max<uint32_t>((rows + 63) / 64 * 64, 64), (uint32_t)std::max(m->max_chunk, 1));
        if ((int)rows > cap) return fail(WICK_CUDA_ERR_BAD_ARG, "batch larger than the model's scratch (" + std::to_string(cap) + " rows)");
        W_TRY(dev_alloc(m, &m->logits_rows, (size_t)cap * m->cfg.vocab_size));
        W_TRY(dev_alloc(m, &m->rows_tok, (size_t)cap));
        W_TRY(dev_alloc(m, &m->rows_next, (size_t)cap));
        W_TRY(dev_alloc(m, &m->rows_pos, (size_t)cap));
        W_TRY(dev_alloc(m, &m->rows_ptrs, nl * 2 * cap));
        m->batch_cap = cap;
        m->rows_out_cap = 0;
    }
    if (m->tc_built && !m->embd_q6k && !m->tc_embd.q && rows >= 16) {
        // the vocabulary head of a batched step is a 64-row GEMM: worth a tensor-core copy of the matrix
        TcWeight* t = &m->tc_embd;
        t->m_pad = (m->embd.m + 127) / 128 * 128;
        t->m = m->embd.m;
        t->k = m->embd.k;
        W_TRY(dev_alloc(m, &t->q, t->q_bytes()));
        W_TRY(dev_alloc(m, &t->scales_t, t->s_bytes() / sizeof(float)));
        CU_TRY(tc_weight_fill(m->stream, m->embd, t));
        CU_TRY(cudaStreamSynchronize(m->stream));
    }
    const size_t out_need = (size_t)steps * rows;
    if (out_need > m->rows_out_cap) {
        W_TRY(dev_alloc(m, &m->rows_out, out_need));
        m->rows_out_cap = out_need;
    }
    const size_t host_need = (size_t)m->batch_cap * (8 + nl * 16) + out_need * 4 + 64;
    if (host_need > m->h_rows_bytes) {
        if (m->h_rows) cudaFreeHost(m->h_rows);
        m->h_rows = nullptr;
        m->h_rows_bytes = 0;
        CU_TRY(cudaMallocHost((void**)&m->h_rows, host_need));
        m->h_rows_bytes = host_need;
    }
    return WICK_CUDA_OK;
}

// One decode step for n rows: tokens in m->rows_tok, positions in m->rows_pos, per-row state pointers in m->rows_ptrs
// (run_layers, lfm2.rs:1020-1124, for every row; the mat-vecs as batched GEMMs, bit-identical to the mat-vec per row,
// simd.rs:1440-1623).  Leaves the logits of every row in m->logits_rows.
int32_t enqueue_decode_rows(wick_cuda_model* m, int n) {
    cudaStream_t st = m->stream;
    const int hs = m->cfg.hidden_size, is = m->cfg.intermediate_size, hd = m->head_dim, cap = m->batch_cap;
    const float eps = m->cfg.rms_norm_eps;
    auto gemms = [&](std::initializer_list<GemmTarget> list) { run_gemms(m, n, list); };
    embed_rows(m, m->rows_tok, nullptr, n);
    const float* pending = nullptr;
    for (size_t li = 0; li < m->layers.size(); li++) {
        Layer& L = m->layers[li];
        float** p0 = m->rows_ptrs + (li * 2) * cap;
        float** p1 = m->rows_ptrs + (li * 2 + 1) * cap;
        launch_add_rmsnorm_quant(st, m->hidden, pending, L.attn_norm, eps, n, hs, m->q8s, m->q8q, nullptr);
        if (!L.is_attn) {
            gemms({{&L.in_proj, &L.tc_in_proj, m->proj}});
            launch_shortconv_rows(st, m->proj, L.conv_w, p0, n, hs, m->cfg.conv_kernel_size, m->q8s, m->q8q);
            gemms({{&L.out_proj, &L.tc_out_proj, m->block_out}});
        } else {
            gemms({{&L.q, &L.tc_q, m->qbuf}, {&L.k, &L.tc_k, m->kbuf}, {&L.v, &L.tc_v, m->vbuf}});
            launch_qknorm_rope_kv_rows(st, m->qbuf, m->kbuf, m->vbuf, L.q_norm, L.k_norm, eps, m->rope_cos, m->rope_sin, p0, p1, m->rows_pos, n,
                                       m->cfg.n_heads, L.n_kv, hd);
            if (m->attn_splitk)
                launch_attention_splitk(st, m->qbuf, p0, p1, nullptr, nullptr, m->rows_pos, m->attn_out, m->splitk_scratch, n, m->cfg.n_heads, L.n_kv,
                                        hd, m->cfg.max_seq_len);
            else
                CU_TRY(launch_attention_rows(st, m->qbuf, p0, p1, m->rows_pos, m->attn_out, n, m->cfg.n_heads, L.n_kv, hd, m->cfg.max_seq_len));
            launch_quant_rows(st, m->attn_out, n, hs, m->q8s, m->q8q);
            gemms({{&L.o, &L.tc_o, m->block_out}});
        }
        launch_add_rmsnorm_quant(st, m->hidden, m->block_out, L.ffn_norm, eps, n, hs, m->q8s, m->q8q, nullptr);
        gemms({{&L.gate, &L.tc_gate, m->gate}, {&L.up, &L.tc_up, m->up}});
        launch_silu_mul_quant(st, m->gate, m->up, n, is, m->q8s, m->q8q, nullptr);
        gemms({{&L.down, &L.tc_down, m->ffn_out}});
        pending = m->ffn_out;
    }
    launch_add_rmsnorm_quant(st, m->hidden, pending, m->output_norm, eps, n, hs, m->q8s, m->q8q, nullptr);
    if (m->embd_q6k) {
        for (int j = 0; j < n; j++)
            launch_gemv_q6k(st, m->embd6, m->q8s + (size_t)j * (hs / QK), m->q8q + (size_t)j * hs, m->logits_rows + (size_t)j * m->cfg.vocab_size);
    } else if (m->tc_embd.q) {
        gemms({{&m->embd, &m->tc_embd, m->logits_rows}});
    } else {
        launch_gemm(st, m->embd, m->q8s, m->q8q, n, m->logits_rows);
    }
    return WICK_CUDA_OK;
}

// Shared driver of the batched entry points: n_steps greedy steps for the rows, or (logits_host != NULL) one step
// that returns every row's logits instead of feeding the argmax back.
int32_t decode_rows(wick_cuda_model* m, const uint32_t* tokens_host, const uint32_t* seq_ids_host, uint32_t bs, uint32_t n_steps,
                    uint32_t* out_tokens_host, float* logits_host) {
    W_TRY(check_model(m));
    if (bs == 0 || n_steps == 0) return WICK_CUDA_OK;
    if (!tokens_host || !seq_ids_host || (!out_tokens_host && !logits_host)) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (bs > MAX_BATCH_ROWS) return fail(WICK_CUDA_ERR_BAD_ARG, "batch of " + std::to_string(bs) + " rows exceeds " + std::to_string(MAX_BATCH_ROWS));
    std::vector<uint8_t> seen(m->seqs.size(), 0);
    for (uint32_t j = 0; j < bs; j++) {
        W_TRY(check_seq(m, seq_ids_host[j]));
        if (seen[seq_ids_host[j]]) return fail(WICK_CUDA_ERR_BAD_ARG, "sequence " + std::to_string(seq_ids_host[j]) + " appears twice in one batch");
        seen[seq_ids_host[j]] = 1;
        if (tokens_host[j] >= m->cfg.vocab_size)
            return fail(WICK_CUDA_ERR_BAD_ARG, "token_id " + std::to_string(tokens_host[j]) + " out of range (vocab_size=" + std::to_string(m->cfg.vocab_size) + ")");
        if ((uint64_t)m->seqs[seq_ids_host[j]].seq_len + n_steps > m->cfg.max_seq_len)
            return fail(WICK_CUDA_ERR_CONTEXT_FULL, "sequence " + std::to_string(seq_ids_host[j]) + ": seq_len + steps exceeds max_seq_len " +
                                                        std::to_string(m->cfg.max_seq_len));
    }
    CU_TRY(cudaSetDevice(m->device));
    if (bs >= 16) W_TRY(ensure_tc(m));
    if (m->attn_splitk) W_TRY(ensure_splitk_scratch(m, (int)bs));
    W_TRY(ensure_batch_buffers(m, bs, n_steps));
    const size_t nl = m->layers.size();
    const int cap = m->batch_cap;
    // staging: tokens, positions, then the per-layer pointer table
    uint32_t* h_tok = (uint32_t*)m->h_rows;
    uint32_t* h_pos = h_tok + cap;
    float** h_ptr = (float**)(m->h_rows + (size_t)cap * 8);
    uint32_t* h_out = (uint32_t*)(m->h_rows + (size_t)cap * (8 + nl * 16));
    for (uint32_t j = 0; j < bs; j++) {
        const wick_cuda_model::SeqSlot& sl = m->seqs[seq_ids_host[j]];
        h_tok[j] = tokens_host[j];
        h_pos[j] = sl.seq_len;
        for (size_t li = 0; li < nl; li++) {
            h_ptr[(li * 2) * cap + j] = m->layers[li].is_attn ? sl.k_cache[li] : sl.conv_state[li];
            h_ptr[(li * 2 + 1) * cap + j] = m->layers[li].is_attn ? sl.v_cache[li] : nullptr;
        }
    }
    CU_TRY(cudaEventRecord(m->ev0, m->stream));
    CU_TRY(cudaMemcpyAsync(m->rows_tok, h_tok, (size_t)bs * 4, cudaMemcpyHostToDevice, m->stream));
    CU_TRY(cudaMemcpyAsync(m->rows_pos, h_pos, (size_t)bs * 4, cudaMemcpyHostToDevice, m->stream));
    CU_TRY(cudaMemcpyAsync(m->rows_ptrs, h_ptr, nl * 2 * cap * sizeof(float*), cudaMemcpyHostToDevice, m->stream));
    const unsigned long long before = g_kernel_launches;
    for (uint32_t s_i = 0; s_i < n_steps; s_i++) {
        W_TRY(enqueue_decode_rows(m, (int)bs));
        if (!logits_host) {
            launch_argmax_rows(m->stream, m->logits_rows, (int)bs, (int)m->cfg.vocab_size, m->rows_next);
            launch_rows_advance(m->stream, m->rows_tok, m->rows_next, m->rows_pos, m->rows_out, (int)bs, (int)s_i);
        }
    }
    m->launches += g_kernel_launches - before;
    CU_TRY(cudaGetLastError());
    if (!logits_host) CU_TRY(cudaMemcpyAsync(h_out, m->rows_out, (size_t)n_steps * bs * 4, cudaMemcpyDeviceToHost, m->stream));
    m->h_u32[2] = 0;
    if (m->tc_err) CU_TRY(cudaMemcpyAsync(m->h_u32 + 2, m->tc_err, 4, cudaMemcpyDeviceToHost, m->stream));
    CU_TRY(cudaEventRecord(m->ev1, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (m->h_u32[2] != 0) {
        const uint32_t code = m->h_u32[2];
        cudaMemsetAsync(m->tc_err, 0, 4, m->stream);
        return fail(WICK_CUDA_ERR_TIMEOUT, "tensor-core GEMM: a bounded wait expired (role code " + std::to_string(code) + ")");
    }
    if (logits_host)
        CU_TRY(cudaMemcpy(logits_host, m->logits_rows, (size_t)bs * m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost));
    else
        memcpy(out_tokens_host, h_out, (size_t)n_steps * bs * 4);
    for (uint32_t j = 0; j < bs; j++) m->seqs[seq_ids_host[j]].seq_len += n_steps;
    return WICK_CUDA_OK;
}

int32_t pre_step(wick_cuda_model* m, uint32_t token, uint32_t pos) {
    W_TRY(check_model(m));
    if (token >= m->cfg.vocab_size)
        return fail(WICK_CUDA_ERR_BAD_ARG, "token_id " + std::to_string(token) + " out of range (vocab_size=" +
                                               std::to_string(m->cfg.vocab_size) + ")");
    if (pos != m->seq_len)
        return fail(WICK_CUDA_ERR_BAD_ARG, "pos " + std::to_string(pos) + " != model seq_len " + std::to_string(m->seq_len));
    if (m->seq_len >= m->cfg.max_seq_len)
        return fail(WICK_CUDA_ERR_CONTEXT_FULL, "seq_len " + std::to_string(m->seq_len) + " reached max_seq_len " +
                                                    std::to_string(m->cfg.max_seq_len));
    CU_TRY(cudaSetDevice(m->device));
    return WICK_CUDA_OK;
}

}  // namespace

// ── C ABI ──────────────────────────────────────────────────────────────────
extern "C" {

int32_t wick_cuda_device_count(int32_t* count) {
    if (!count) return fail(WICK_CUDA_ERR_BAD_ARG, "count is NULL");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        return fail(WICK_CUDA_ERR_CUDA, std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e));
    }
    *count = n;
    return WICK_CUDA_OK;
}

const char* wick_cuda_last_error(void) { return g_last_error.c_str(); }

int32_t wick_cuda_model_create(const uint8_t* gguf_host, size_t gguf_len, uint32_t context_size, int32_t device,
                               wick_cuda_model** out) {
    if (!gguf_host || !out) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    *out = nullptr;
    std::unique_ptr<GgufImage> img;
    try {
        img.reset(new GgufImage(gguf_host, gguf_len));
    } catch (const std::exception& e) {
        return fail(WICK_CUDA_ERR_BAD_GGUF, e.what());
    }
    int ndev = 0;
    CU_TRY(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(WICK_CUDA_ERR_BAD_ARG, "no such CUDA device: " + std::to_string(device));
    CU_TRY(cudaSetDevice(device));
    std::unique_ptr<wick_cuda_model> m(new wick_cuda_model());
    m->device = device;
    int32_t r = build_model(m.get(), *img, context_size);
    if (r != WICK_CUDA_OK) return r;
    *out = m.release();
    return WICK_CUDA_OK;
}

int32_t wick_cuda_model_create_from_file(const char* path, uint32_t context_size, int32_t device, wick_cuda_model** out) {
    if (!path || !out) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) return fail(WICK_CUDA_ERR_BAD_GGUF, std::string("cannot open ") + path);
    std::streamsize len = f.tellg();
    f.seekg(0);
    std::vector<uint8_t> buf((size_t)len);
    if (len > 0 && !f.read((char*)buf.data(), len)) return fail(WICK_CUDA_ERR_BAD_GGUF, std::string("cannot read ") + path);
    return wick_cuda_model_create(buf.data(), buf.size(), context_size, device, out);
}

void wick_cuda_model_destroy(wick_cuda_model* m) { delete m; }

int32_t wick_cuda_model_config(const wick_cuda_model* m, wick_cuda_config* out) {
    W_TRY(check_model(m));
    if (!out) return fail(WICK_CUDA_ERR_BAD_ARG, "out is NULL");
    *out = m->cfg;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_model_kv_heads_per_layer(const wick_cuda_model* m, uint32_t* out, uint32_t n) {
    W_TRY(check_model(m));
    if (!out || n != m->cfg.n_layers) return fail(WICK_CUDA_ERR_BAD_ARG, "out is NULL or n != n_layers");
    for (uint32_t i = 0; i < n; i++) out[i] = m->layers[i].is_attn ? m->layers[i].n_kv : 0;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_gpu_memory_bytes(const wick_cuda_model* m, uint64_t* out) {
    W_TRY(check_model(m));
    if (!out) return fail(WICK_CUDA_ERR_BAD_ARG, "out is NULL");
    *out = m->bytes;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_forward(wick_cuda_model* m, uint32_t token, uint32_t pos, float* logits_host) {
    W_TRY(pre_step(m, token, pos));
    if (!logits_host) return fail(WICK_CUDA_ERR_BAD_ARG, "logits_host is NULL");
    m->h_u32[0] = token;
    CU_TRY(cudaEventRecord(m->ev0, m->stream));
    CU_TRY(cudaMemcpyAsync(&m->ctl->token, m->h_u32, 4, cudaMemcpyHostToDevice, m->stream));
    if (m->mega_ok) {
        W_TRY(run_mega(m, 1, false));
    } else {
        CU_TRY(cudaGraphLaunch(m->g_logits, m->stream));
        m->launches += m->nodes_logits;
    }
    CU_TRY(cudaMemcpyAsync(m->h_logits, m->logits, (size_t)m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, m->stream));
    CU_TRY(cudaEventRecord(m->ev1, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (m->mega_ok) W_TRY(check_mega_status(m));
    memcpy(logits_host, m->h_logits, (size_t)m->cfg.vocab_size * 4);
    m->seq_len += 1;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_forward_greedy(wick_cuda_model* m, uint32_t token, uint32_t pos, uint32_t* next_token) {
    W_TRY(pre_step(m, token, pos));
    if (!next_token) return fail(WICK_CUDA_ERR_BAD_ARG, "next_token is NULL");
    m->h_u32[0] = token;
    CU_TRY(cudaEventRecord(m->ev0, m->stream));
    CU_TRY(cudaMemcpyAsync(&m->ctl->token, m->h_u32, 4, cudaMemcpyHostToDevice, m->stream));
    if (m->mega_ok) {
        W_TRY(run_mega(m, 1, true));  // copies the control block (with the chosen token) back
    } else {
        CU_TRY(cudaGraphLaunch(m->g_greedy, m->stream));
        m->launches += m->nodes_greedy;
        CU_TRY(cudaMemcpyAsync(m->h_u32 + 1, m->argmax_tok, 4, cudaMemcpyDeviceToHost, m->stream));
    }
    CU_TRY(cudaEventRecord(m->ev1, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (m->mega_ok) {
        W_TRY(check_mega_status(m));
        m->h_u32[1] = m->h_ctl->token;
    }
    *next_token = m->h_u32[1];
    m->seq_len += 1;
    return WICK_CUDA_OK;
}

// Model::forward followed by Sampler::sample (sampler.rs:64-158) on the device: the logits never leave the GPU.
int32_t wick_cuda_forward_sample(wick_cuda_model* m, uint32_t token, uint32_t pos, float temperature, uint32_t top_k, float top_p, float r,
                                 uint32_t* next_token) {
    W_TRY(pre_step(m, token, pos));
    if (!next_token) return fail(WICK_CUDA_ERR_BAD_ARG, "next_token is NULL");
    if (temperature <= 0.0f || top_k == 1) return wick_cuda_forward_greedy(m, token, pos, next_token);  // sampler.rs:71-73
    if (top_p < 1.0f && (top_k == 0 || top_k > 4096))
        return fail(WICK_CUDA_ERR_BAD_ARG, "on-device top-p needs 1 <= top_k <= 4096 (read the logits back and sample on the host instead)");
    if (!m->sample_val) {
        W_TRY(dev_alloc(m, &m->sample_val, (size_t)m->cfg.vocab_size));
        W_TRY(dev_alloc(m, &m->sample_idx, (size_t)m->cfg.vocab_size));
        W_TRY(dev_alloc(m, &m->sample_status, 1));
        CU_TRY(cudaMemset(m->sample_status, 0, 4));
    }
    m->h_u32[0] = token;
    CU_TRY(cudaEventRecord(m->ev0, m->stream));
    CU_TRY(cudaMemcpyAsync(&m->ctl->token, m->h_u32, 4, cudaMemcpyHostToDevice, m->stream));
    if (m->mega_ok) {
        W_TRY(run_mega(m, 1, false));
    } else {
        CU_TRY(cudaGraphLaunch(m->g_logits, m->stream));
        m->launches += m->nodes_logits;
    }
    launch_sample(m->stream, m->logits, (int)m->cfg.vocab_size, temperature, (int)top_k, top_p, r, m->sample_val, m->sample_idx, m->argmax_tok,
                  m->sample_status);
    m->launches += 1;
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(m->h_u32 + 1, m->argmax_tok, 4, cudaMemcpyDeviceToHost, m->stream));
    CU_TRY(cudaMemcpyAsync(m->h_u32 + 2, m->sample_status, 4, cudaMemcpyDeviceToHost, m->stream));
    CU_TRY(cudaEventRecord(m->ev1, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (m->mega_ok) W_TRY(check_mega_status(m));
    m->seq_len += 1;  // the step itself has run
    if (m->h_u32[2]) {
        cudaMemsetAsync(m->sample_status, 0, 4, m->stream);
        return fail(WICK_CUDA_ERR_BAD_ARG, "on-device top-p: more than 4096 logits tie at or above the top-k threshold");
    }
    *next_token = m->h_u32[1];
    return WICK_CUDA_OK;
}

int32_t wick_cuda_generate_greedy(wick_cuda_model* m, uint32_t first_token, uint32_t n_steps, uint32_t* out_tokens_host) {
    W_TRY(check_model(m));
    if (n_steps == 0) return WICK_CUDA_OK;
    W_TRY(pre_step(m, first_token, m->seq_len));
    if (!out_tokens_host) return fail(WICK_CUDA_ERR_BAD_ARG, "out_tokens_host is NULL");
    if ((uint64_t)m->seq_len + n_steps > m->cfg.max_seq_len)
        return fail(WICK_CUDA_ERR_CONTEXT_FULL, "seq_len + n_steps exceeds max_seq_len " + std::to_string(m->cfg.max_seq_len));
    // token and ring cursor for this run
    uint32_t init[3] = {first_token, m->seq_len, 0};
    memcpy(m->h_u32, init, sizeof(init));
    CU_TRY(cudaEventRecord(m->ev0, m->stream));
    CU_TRY(cudaMemcpyAsync(m->ctl, m->h_u32, sizeof(init), cudaMemcpyHostToDevice, m->stream));
    if (m->mega_ok) {
        W_TRY(run_mega(m, (int)n_steps, true));
    } else {
        for (uint32_t i = 0; i < n_steps; i++) CU_TRY(cudaGraphLaunch(m->g_greedy, m->stream));
        m->launches += m->nodes_greedy * n_steps;
    }
    CU_TRY(cudaMemcpyAsync(m->h_u32, m->ring, (size_t)n_steps * 4, cudaMemcpyDeviceToHost, m->stream));
    CU_TRY(cudaEventRecord(m->ev1, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (m->mega_ok) W_TRY(check_mega_status(m));
    memcpy(out_tokens_host, m->h_u32, (size_t)n_steps * 4);
    m->seq_len += n_steps;
    return WICK_CUDA_OK;
}

// forward_prefill and its embedding-input relatives: exactly one of tokens_host / emb_host is given; the
// result is the logits of the last position (logits_host) and / or its output-normed hidden row (hidden_host).
static int32_t prefill_core(wick_cuda_model* m, const uint32_t* tokens_host, const float* emb_host, uint32_t n, uint32_t start_pos,
                            float* logits_host, float* hidden_host) {
    const int hs = m->cfg.hidden_size;
    if (n == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "forward_prefill requires at least one token");
    if (tokens_host)
        for (uint32_t i = 0; i < n; i++)
            if (tokens_host[i] >= m->cfg.vocab_size)
                return fail(WICK_CUDA_ERR_BAD_ARG, "token_id " + std::to_string(tokens_host[i]) + " out of range for vocab size " +
                                                       std::to_string(m->cfg.vocab_size));
    if (start_pos != 0 && start_pos != m->seq_len)
        return fail(WICK_CUDA_ERR_BAD_ARG, "start_pos " + std::to_string(start_pos) + " != model seq_len " + std::to_string(m->seq_len));
    if ((uint64_t)start_pos + n > m->cfg.max_seq_len)
        return fail(WICK_CUDA_ERR_CONTEXT_FULL, "start_pos + n = " + std::to_string((uint64_t)start_pos + n) +
                                                    " exceeds max_seq_len " + std::to_string(m->cfg.max_seq_len));
    CU_TRY(cudaSetDevice(m->device));
    if (n >= 16) W_TRY(ensure_tc(m));
    if (start_pos == 0) W_TRY(reset_sequence(m));  // new sequence, metal_lfm2.rs:2361-2397
    const bool flash = n >= 256;  // FLASH_ATTN_THRESHOLD, lfm2.rs:1646-1647
    CU_TRY(cudaEventRecord(m->ev0, m->stream));
    for (uint32_t c0 = 0; c0 < n; c0 += m->max_chunk) {
        uint32_t cn = std::min<uint32_t>(m->max_chunk, n - c0);
        if (tokens_host) {
            memcpy(m->h_u32, tokens_host + c0, (size_t)cn * 4);
            CU_TRY(cudaMemcpyAsync(m->tokens_dev, m->h_u32, (size_t)cn * 4, cudaMemcpyHostToDevice, m->stream));
        } else {
            CU_TRY(cudaMemcpyAsync(m->hidden, emb_host + (size_t)c0 * hs, (size_t)cn * hs * 4, cudaMemcpyHostToDevice, m->stream));
        }
        const unsigned long long before = g_kernel_launches;
        enqueue_prefill_chunk(m, (int)cn, (int)(start_pos + c0), flash, c0 + cn == n, tokens_host != nullptr, logits_host != nullptr);
        m->launches += g_kernel_launches - before;
        CU_TRY(cudaGetLastError());
        CU_TRY(cudaStreamSynchronize(m->stream));  // h_u32 is reused by the next chunk
        prof_collect(m);
    }
    uint32_t newpos[2] = {0, start_pos + n};
    memcpy(m->h_u32, newpos, 8);
    CU_TRY(cudaMemcpyAsync(&m->ctl->pos, m->h_u32 + 1, 4, cudaMemcpyHostToDevice, m->stream));
    if (logits_host) CU_TRY(cudaMemcpyAsync(m->h_logits, m->logits, (size_t)m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, m->stream));
    m->h_u32[2] = 0;
    if (m->tc_err) CU_TRY(cudaMemcpyAsync(m->h_u32 + 2, m->tc_err, 4, cudaMemcpyDeviceToHost, m->stream));
    CU_TRY(cudaEventRecord(m->ev1, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (m->h_u32[2] != 0) {
        const uint32_t code = m->h_u32[2];
        cudaMemsetAsync(m->tc_err, 0, 4, m->stream);
        return fail(WICK_CUDA_ERR_TIMEOUT, "prefill kernel (tensor-core GEMM or tiled attention): a bounded wait expired (code " + std::to_string(code) + ")");
    }
    if (logits_host) memcpy(logits_host, m->h_logits, (size_t)m->cfg.vocab_size * 4);
    if (hidden_host) CU_TRY(cudaMemcpy(hidden_host, m->normed_last, (size_t)hs * 4, cudaMemcpyDeviceToHost));
    m->seq_len = start_pos + n;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_forward_prefill(wick_cuda_model* m, const uint32_t* tokens_host, uint32_t n, uint32_t start_pos,
                                  float* logits_host) {
    W_TRY(check_model(m));
    if (!tokens_host || !logits_host) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    return prefill_core(m, tokens_host, nullptr, n, start_pos, logits_host, nullptr);
}

int32_t wick_cuda_forward_prefill_from_embeddings(wick_cuda_model* m, const float* embeddings_host, uint32_t n, uint32_t start_pos,
                                                  float* logits_host) {
    W_TRY(check_model(m));
    if (!embeddings_host || !logits_host) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (n == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "forward_prefill_from_embeddings requires at least one frame");
    return prefill_core(m, nullptr, embeddings_host, n, start_pos, logits_host, nullptr);
}

// The single-step embedding-input methods run the one-row prefill pipeline at the model's own
// position (like forward, they ignore `pos`); a one-row prefill is bit-identical to a decode step.
int32_t wick_cuda_forward_from_embedding(wick_cuda_model* m, const float* embedding_host, uint32_t pos, float* logits_host) {
    (void)pos;
    W_TRY(check_model(m));
    if (!embedding_host || !logits_host) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    return prefill_core(m, nullptr, embedding_host, 1, m->seq_len, logits_host, nullptr);
}

int32_t wick_cuda_forward_hidden_from_embedding(wick_cuda_model* m, const float* embedding_host, uint32_t pos, float* hidden_host) {
    (void)pos;
    W_TRY(check_model(m));
    if (!embedding_host || !hidden_host) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    return prefill_core(m, nullptr, embedding_host, 1, m->seq_len, nullptr, hidden_host);
}

int32_t wick_cuda_forward_embedding(wick_cuda_model* m, uint32_t token, uint32_t pos, float* hidden_host) {
    (void)pos;
    W_TRY(check_model(m));
    if (!hidden_host) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    return prefill_core(m, &token, nullptr, 1, m->seq_len, nullptr, hidden_host);
}

// Model::shift_kv (mod.rs:158-170; lfm2.rs:2507-2516 -> kv_cache.rs:601-715).
int32_t wick_cuda_shift_kv(wick_cuda_model* m, uint32_t n_keep, uint32_t shift) {
    W_TRY(check_model(m));
    if (shift == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "shift must be > 0");
    if ((uint64_t)n_keep + shift > m->seq_len)
        return fail(WICK_CUDA_ERR_BAD_ARG, "shift range out of bounds: n_keep=" + std::to_string(n_keep) + " + shift=" +
                                               std::to_string(shift) + " > seq_len=" + std::to_string(m->seq_len));
    CU_TRY(cudaSetDevice(m->device));
    const int hd = m->head_dim, half = hd / 2;
    const uint32_t new_len = m->seq_len - shift;
    const int retained = (int)(new_len - n_keep);
    if (retained > 0) {
        // delta rotation table with the host libm in the reference's order (cpu.rs:2174-2187)
        std::vector<float> tab(hd);
        const float theta_scale = powf(m->cfg.rope_theta, -2.0f / (float)hd);
        float theta = (float)(-(int)shift);
        for (int i = 0; i < half; i++) {
            tab[i] = cosf(theta);
            tab[half + i] = sinf(theta);
            theta *= theta_scale;
        }
        CU_TRY(cudaMemcpyAsync(m->rope_delta, tab.data(), (size_t)hd * 4, cudaMemcpyHostToDevice, m->stream));
        CU_TRY(cudaStreamSynchronize(m->stream));  // `tab` is pageable host memory
        const size_t scratch_floats = (size_t)m->max_chunk * m->cfg.intermediate_size;
        const unsigned long long before = g_kernel_launches;
        for (Layer& L : m->layers) {
            if (!L.is_attn) continue;
            const int kv_dim = L.n_kv * hd;
            const int rows_per_pass = (int)std::max<size_t>(1, scratch_floats / kv_dim);
            // ascending passes: a pass only overwrites rows below the ones later passes still have to read
            for (int r0 = 0; r0 < retained; r0 += rows_per_pass) {
                const int rows = std::min(rows_per_pass, retained - r0);
                const int row0 = (int)n_keep + r0;
                launch_kv_shift_gather(m->stream, L.k_cache, m->gate, row0, rows, (int)shift, kv_dim, hd, m->rope_delta, m->rope_delta + half);
                launch_kv_shift_gather(m->stream, L.v_cache, m->up, row0, rows, (int)shift, kv_dim, hd, nullptr, nullptr);
                CU_TRY(cudaMemcpyAsync(L.k_cache + (size_t)row0 * kv_dim, m->gate, (size_t)rows * kv_dim * 4, cudaMemcpyDeviceToDevice, m->stream));
                CU_TRY(cudaMemcpyAsync(L.v_cache + (size_t)row0 * kv_dim, m->up, (size_t)rows * kv_dim * 4, cudaMemcpyDeviceToDevice, m->stream));
            }
        }
        m->launches += g_kernel_launches - before;
        CU_TRY(cudaGetLastError());
    }
    m->h_u32[0] = new_len;
    CU_TRY(cudaMemcpyAsync(&m->ctl->pos, m->h_u32, 4, cudaMemcpyHostToDevice, m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    m->seq_len = new_len;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_set_prefill_mode(wick_cuda_model* m, int32_t mode) {
    W_TRY(check_model(m));
    if (mode != WICK_CUDA_PREFILL_EXACT && mode != WICK_CUDA_PREFILL_TENSOR && mode != WICK_CUDA_PREFILL_EXACT_CUDA_CORES)
        return fail(WICK_CUDA_ERR_BAD_ARG, "unknown prefill mode " + std::to_string(mode));
    if (mode == WICK_CUDA_PREFILL_TENSOR && !m->tc_ok)
        return fail(WICK_CUDA_ERR_BAD_ARG, "tensor-core prefill needs hidden and feed-forward sizes that are multiples of 128");
    m->prefill_mode = mode;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_prefill_mode(const wick_cuda_model* m, int32_t* mode) {
    W_TRY(check_model(m));
    if (!mode) return fail(WICK_CUDA_ERR_BAD_ARG, "mode is NULL");
    *mode = m->prefill_mode;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_prefill_uses_tensor_cores(const wick_cuda_model* m, int32_t* yes) {
    W_TRY(check_model(m));
    if (!yes) return fail(WICK_CUDA_ERR_BAD_ARG, "yes is NULL");
    *yes = m->tc_ok && m->prefill_mode != WICK_CUDA_PREFILL_EXACT_CUDA_CORES;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_reset(wick_cuda_model* m) {
    W_TRY(check_model(m));
    CU_TRY(cudaSetDevice(m->device));
    return reset_sequence(m);
}

int32_t wick_cuda_seq_len(const wick_cuda_model* m, uint32_t* out) {
    W_TRY(check_model(m));
    if (!out) return fail(WICK_CUDA_ERR_BAD_ARG, "out is NULL");
    *out = m->seq_len;
    return WICK_CUDA_OK;
}

// snapshot image: u32 magic, u32 seq_len, then per layer either K rows + V rows (seq_len x
// kv_dim f32 each) or the conv buffer (d_conv x hidden f32)
static const uint32_t SNAP_MAGIC = 0x534B4357u;  // "WCKS"

int32_t wick_cuda_snapshot_size(const wick_cuda_model* m, uint64_t* bytes) {
    W_TRY(check_model(m));
    if (!bytes) return fail(WICK_CUDA_ERR_BAD_ARG, "bytes is NULL");
    uint64_t b = 8;
    const int dc = (int)m->cfg.conv_kernel_size - 1;
    for (const Layer& L : m->layers)
        b += L.is_attn ? (uint64_t)2 * m->seq_len * L.n_kv * m->head_dim * 4 : (uint64_t)dc * m->cfg.hidden_size * 4;
    *bytes = b;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_snapshot(wick_cuda_model* m, uint8_t* out_host, uint64_t capacity) {
    uint64_t need = 0;
    W_TRY(wick_cuda_snapshot_size(m, &need));
    if (!out_host || capacity < need) return fail(WICK_CUDA_ERR_BAD_ARG, "snapshot buffer too small");
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaStreamSynchronize(m->stream));
    uint32_t head[2] = {SNAP_MAGIC, m->seq_len};
    memcpy(out_host, head, 8);
    uint8_t* p = out_host + 8;
    const int dc = (int)m->cfg.conv_kernel_size - 1;
    for (const Layer& L : m->layers) {
        if (L.is_attn) {
            size_t b = (size_t)m->seq_len * L.n_kv * m->head_dim * 4;
            if (b) {
                CU_TRY(cudaMemcpy(p, L.k_cache, b, cudaMemcpyDeviceToHost));
                CU_TRY(cudaMemcpy(p + b, L.v_cache, b, cudaMemcpyDeviceToHost));
            }
            p += 2 * b;
        } else {
            size_t b = (size_t)dc * m->cfg.hidden_size * 4;
            if (b) CU_TRY(cudaMemcpy(p, L.conv_state, b, cudaMemcpyDeviceToHost));
            p += b;
        }
    }
    return WICK_CUDA_OK;
}

int32_t wick_cuda_restore(wick_cuda_model* m, const uint8_t* snap_host, uint64_t len) {
    W_TRY(check_model(m));
    if (!snap_host || len < 8) return fail(WICK_CUDA_ERR_BAD_ARG, "snapshot too short");
    uint32_t head[2];
    memcpy(head, snap_host, 8);
    if (head[0] != SNAP_MAGIC) return fail(WICK_CUDA_ERR_BAD_ARG, "not a wick_cuda snapshot");
    if (head[1] > m->cfg.max_seq_len) return fail(WICK_CUDA_ERR_CONTEXT_FULL, "snapshot longer than max_seq_len");
    uint32_t saved = m->seq_len;
    m->seq_len = head[1];
    uint64_t need = 0;
    wick_cuda_snapshot_size(m, &need);
    if (need != len) {
        m->seq_len = saved;
        return fail(WICK_CUDA_ERR_BAD_ARG, "snapshot size does not match this model");
    }
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaStreamSynchronize(m->stream));
    const uint8_t* p = snap_host + 8;
    const int dc = (int)m->cfg.conv_kernel_size - 1;
    for (const Layer& L : m->layers) {
        if (L.is_attn) {
            size_t b = (size_t)m->seq_len * L.n_kv * m->head_dim * 4;
            if (b) {
                CU_TRY(cudaMemcpy(L.k_cache, p, b, cudaMemcpyHostToDevice));
                CU_TRY(cudaMemcpy(L.v_cache, p + b, b, cudaMemcpyHostToDevice));
            }
            p += 2 * b;
        } else {
            size_t b = (size_t)dc * m->cfg.hidden_size * 4;
            if (b) CU_TRY(cudaMemcpy(L.conv_state, p, b, cudaMemcpyHostToDevice));
            p += b;
        }
    }
    CU_TRY(cudaMemcpy(&m->ctl->pos, &m->seq_len, 4, cudaMemcpyHostToDevice));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_last_elapsed_ms(wick_cuda_model* m, float* ms) {
    W_TRY(check_model(m));
    if (!ms) return fail(WICK_CUDA_ERR_BAD_ARG, "ms is NULL");
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaEventSynchronize(m->ev1));
    CU_TRY(cudaEventElapsedTime(ms, m->ev0, m->ev1));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_kernel_launches(const wick_cuda_model* m, uint64_t* count) {
    W_TRY(check_model(m));
    if (!count) return fail(WICK_CUDA_ERR_BAD_ARG, "count is NULL");
    *count = m->launches;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_set_decode_attention(wick_cuda_model* m, int32_t mode) {
    W_TRY(check_model(m));
    if (mode != WICK_CUDA_DECODE_ATTENTION_EXACT && mode != WICK_CUDA_DECODE_ATTENTION_SPLITK)
        return fail(WICK_CUDA_ERR_BAD_ARG, "unknown decode attention mode " + std::to_string(mode));
    const bool want = mode == WICK_CUDA_DECODE_ATTENTION_SPLITK;
    if (want == m->attn_splitk) return WICK_CUDA_OK;
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaStreamSynchronize(m->stream));
    if (want) W_TRY(ensure_splitk_scratch(m, std::max(1, m->batch_cap)));
    m->attn_splitk = want;
    // the captured decode graphs contain the attention kernels: capture them again
    if (m->g_logits) cudaGraphExecDestroy(m->g_logits);
    if (m->g_greedy) cudaGraphExecDestroy(m->g_greedy);
    m->g_logits = m->g_greedy = nullptr;
    W_TRY(capture_graph(m, false, &m->g_logits, &m->nodes_logits));
    W_TRY(capture_graph(m, true, &m->g_greedy, &m->nodes_greedy));
    CU_TRY(cudaStreamSynchronize(m->stream));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_profile_enable(wick_cuda_model* m, int32_t on) {
    W_TRY(check_model(m));
    m->prof_on = on != 0;
    for (double& v : m->prof_ms) v = 0.0;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_profile_read(wick_cuda_model* m, double* ms_out, uint32_t capacity) {
    W_TRY(check_model(m));
    if (!ms_out || capacity < WICK_CUDA_PROFILE_CATEGORIES) return fail(WICK_CUDA_ERR_BAD_ARG, "ms_out is NULL or shorter than WICK_CUDA_PROFILE_CATEGORIES");
    for (int i = 0; i < WICK_CUDA_PROFILE_CATEGORIES; i++) ms_out[i] = m->prof_ms[i];
    return WICK_CUDA_OK;
}

const char* wick_cuda_profile_category_name(uint32_t i) { return i < WICK_CUDA_PROFILE_CATEGORIES ? PROF_NAMES[i] : ""; }

int32_t wick_cuda_decode_profile(wick_cuda_model* m, uint64_t* ns_out, int32_t* kinds_out, uint32_t capacity, uint32_t* n_phases) {
    W_TRY(check_model(m));
    if (!m->mega_ok) return fail(WICK_CUDA_ERR_BAD_ARG, "this model decodes through captured graphs");
    if (!n_phases) return fail(WICK_CUDA_ERR_BAD_ARG, "n_phases is NULL");
    const int np = m->last_launch_long ? m->n_phases_long : m->mega.n_phases;
    *n_phases = (uint32_t)np;
    if (!ns_out || !kinds_out || capacity < (uint32_t)np) return WICK_CUDA_OK;
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaStreamSynchronize(m->stream));
    CU_TRY(cudaMemcpy(ns_out, m->d_prof, (size_t)np * 32, cudaMemcpyDeviceToHost));
    if (capacity >= (uint32_t)np + 4)  // optional: the 16 internal stamps of WICK_CUDA_PROF_PHASE
        CU_TRY(cudaMemcpy(ns_out + (size_t)np * 4, m->d_prof + (size_t)np * 4, 128, cudaMemcpyDeviceToHost));
    std::vector<MegaPhase> ph(np);
    CU_TRY(cudaMemcpy(ph.data(), m->last_launch_long ? m->d_phases_long : m->d_phases, ph.size() * sizeof(MegaPhase), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < ph.size(); i++) kinds_out[i] = ph[i].kind;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_debug_skew_barrier(wick_cuda_model* m, int64_t delta) {
    W_TRY(check_model(m));
    if (!m->mega_ok) return fail(WICK_CUDA_ERR_BAD_ARG, "this model decodes through captured graphs");
    m->bar_base = (unsigned long long)((long long)m->bar_base + delta);
    return WICK_CUDA_OK;
}

int32_t wick_cuda_decode_path(const wick_cuda_model* m, int32_t* persistent) {
    W_TRY(check_model(m));
    if (!persistent) return fail(WICK_CUDA_ERR_BAD_ARG, "persistent is NULL");
    *persistent = m->mega_ok ? 1 : 0;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_read_kv(wick_cuda_model* m, uint32_t layer, float* k_host, float* v_host) {
    W_TRY(check_model(m));
    if (layer >= m->layers.size() || !m->layers[layer].is_attn) return fail(WICK_CUDA_ERR_BAD_ARG, "not an attention layer");
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaStreamSynchronize(m->stream));
    const Layer& L = m->layers[layer];
    size_t b = (size_t)m->seq_len * L.n_kv * m->head_dim * 4;
    if (b && k_host) CU_TRY(cudaMemcpy(k_host, L.k_cache, b, cudaMemcpyDeviceToHost));
    if (b && v_host) CU_TRY(cudaMemcpy(v_host, L.v_cache, b, cudaMemcpyDeviceToHost));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_read_conv_state(wick_cuda_model* m, uint32_t layer, float* out_host) {
    W_TRY(check_model(m));
    if (layer >= m->layers.size() || m->layers[layer].is_attn || !out_host) return fail(WICK_CUDA_ERR_BAD_ARG, "not a conv layer");
    CU_TRY(cudaSetDevice(m->device));
    CU_TRY(cudaStreamSynchronize(m->stream));
    size_t b = (size_t)((int)m->cfg.conv_kernel_size - 1) * m->cfg.hidden_size * 4;
    if (b) CU_TRY(cudaMemcpy(out_host, m->layers[layer].conv_state, b, cudaMemcpyDeviceToHost));
    return WICK_CUDA_OK;
}

// ── sequence slots (extension; not reachable from wick's Model trait) ──────

int32_t wick_cuda_seq_create(wick_cuda_model* m, uint32_t* seq_id) {
    W_TRY(check_model(m));
    if (!seq_id) return fail(WICK_CUDA_ERR_BAD_ARG, "seq_id is NULL");
    CU_TRY(cudaSetDevice(m->device));
    size_t id = 0;
    while (id < m->seqs.size() && m->seqs[id].live) id++;
    const int hs = m->cfg.hidden_size, dc = (int)m->cfg.conv_kernel_size - 1;
    if (id == m->seqs.size()) {
        if (m->seqs.size() >= 65536) return fail(WICK_CUDA_ERR_BAD_ARG, "too many sequence slots");
        wick_cuda_model::SeqSlot sl;
        const size_t nl = m->layers.size();
        sl.k_cache.assign(nl, nullptr);
        sl.v_cache.assign(nl, nullptr);
        sl.conv_state.assign(nl, nullptr);
        for (size_t li = 0; li < nl; li++) {
            const Layer& L = m->layers[li];
            if (L.is_attn) {
                const size_t rows = (size_t)m->cfg.max_seq_len * L.n_kv * m->head_dim;
                W_TRY(dev_alloc(m, &sl.k_cache[li], rows));
                W_TRY(dev_alloc(m, &sl.v_cache[li], rows));
            } else {
                W_TRY(dev_alloc(m, &sl.conv_state[li], (size_t)std::max(dc, 1) * hs));
            }
        }
        m->seqs.push_back(std::move(sl));
    }
    wick_cuda_model::SeqSlot& sl = m->seqs[id];  // a recycled slot keeps its buffers
    for (size_t li = 0; li < m->layers.size(); li++)
        if (!m->layers[li].is_attn && dc > 0) CU_TRY(cudaMemsetAsync(sl.conv_state[li], 0, (size_t)dc * hs * sizeof(float), m->stream));
    CU_TRY(cudaStreamSynchronize(m->stream));
    sl.live = true;
    sl.seq_len = 0;
    *seq_id = (uint32_t)id;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_seq_destroy(wick_cuda_model* m, uint32_t seq_id) {
    W_TRY(check_model(m));
    W_TRY(check_seq(m, seq_id));
    m->seqs[seq_id].live = false;  // the buffers stay with the model and serve the next wick_cuda_seq_create
    m->seqs[seq_id].seq_len = 0;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_seq_length(const wick_cuda_model* m, uint32_t seq_id, uint32_t* out) {
    W_TRY(check_model(m));
    W_TRY(check_seq(m, seq_id));
    if (!out) return fail(WICK_CUDA_ERR_BAD_ARG, "out is NULL");
    *out = m->seqs[seq_id].seq_len;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_seq_prefill(wick_cuda_model* m, uint32_t seq_id, const uint32_t* tokens_host, uint32_t n, uint32_t start_pos,
                              float* logits_host) {
    W_TRY(check_model(m));
    W_TRY(check_seq(m, seq_id));
    if (!tokens_host || !logits_host) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    CU_TRY(cudaSetDevice(m->device));
    return with_slot(m, seq_id, [&]() { return prefill_core(m, tokens_host, nullptr, n, start_pos, logits_host, nullptr); });
}

int32_t wick_cuda_decode_batch(wick_cuda_model* m, const uint32_t* tokens_host, const uint32_t* seq_ids_host, uint32_t bs,
                               uint32_t* next_tokens_host) {
    if (!next_tokens_host) return fail(WICK_CUDA_ERR_BAD_ARG, "next_tokens_host is NULL");
    return decode_rows(m, tokens_host, seq_ids_host, bs, 1, next_tokens_host, nullptr);
}

int32_t wick_cuda_decode_batch_steps(wick_cuda_model* m, const uint32_t* first_tokens_host, const uint32_t* seq_ids_host, uint32_t bs,
                                     uint32_t n_steps, uint32_t* out_tokens_host) {
    if (!out_tokens_host) return fail(WICK_CUDA_ERR_BAD_ARG, "out_tokens_host is NULL");
    return decode_rows(m, first_tokens_host, seq_ids_host, bs, n_steps, out_tokens_host, nullptr);
}

int32_t wick_cuda_decode_batch_logits(wick_cuda_model* m, const uint32_t* tokens_host, const uint32_t* seq_ids_host, uint32_t bs,
                                      float* logits_host) {
    if (!logits_host) return fail(WICK_CUDA_ERR_BAD_ARG, "logits_host is NULL");
    return decode_rows(m, tokens_host, seq_ids_host, bs, 1, nullptr, logits_host);
}

// ── operators ──────────────────────────────────────────────────────────────

int32_t wick_cuda_weight_create(int32_t dtype, const uint8_t* raw_host, uint32_t mrows, uint32_t k, wick_cuda_weight** out) {
    if (!raw_host || !out) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    *out = nullptr;
    if (dtype != DT_Q4_0 && dtype != DT_Q8_0) return fail(WICK_CUDA_ERR_UNSUPPORTED_DTYPE, "only Q4_0 (2) and Q8_0 (8) weights are supported");
    if (k == 0 || k % QK || mrows == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "k must be a positive multiple of 32 and m > 0");
    std::unique_ptr<wick_cuda_weight> w(new wick_cuda_weight());
    CU_TRY(cudaGetDevice(&w->device));
    w->w.m = (int)mrows;
    w->w.k = (int)k;
    w->w.dtype = dtype;
    size_t nblk = (size_t)mrows * (k / QK);
    uint8_t *staging = nullptr, *q = nullptr;
    __half* d = nullptr;
    CU_TRY(cudaMalloc((void**)&staging, nblk * 34));
    cudaError_t e1 = cudaMalloc((void**)&q, std::max<size_t>(w->w.q_bytes(), 256));
    cudaError_t e2 = cudaMalloc((void**)&d, std::max<size_t>(w->w.d_bytes(), 256));
    int32_t r = WICK_CUDA_OK;
    if (e1 != cudaSuccess || e2 != cudaSuccess) r = fail(WICK_CUDA_ERR_OOM, "cudaMalloc failed for weight planes");
    if (r == WICK_CUDA_OK) r = upload_weight_raw(w->w, raw_host, staging, nullptr, q, d);
    cudaFree(staging);
    if (r != WICK_CUDA_OK) {
        cudaFree(q);
        cudaFree(d);
        return r;
    }
    w->w.q = q;
    w->w.d = d;
    *out = w.release();
    return WICK_CUDA_OK;
}

void wick_cuda_weight_destroy(wick_cuda_weight* w) {
    if (!w) return;
    cudaFree((void*)w->w.q);
    cudaFree((void*)w->w.d);
    cudaFree(w->tc.q);
    cudaFree(w->tc.scales_t);
    cudaFree(w->tc_err);
    delete w;
}

#define OP_END()                  \
    CU_TRY(cudaGetLastError());   \
    return WICK_CUDA_OK

int32_t wick_cuda_quantize_q8_0(const float* x_dev, uint32_t n, uint32_t k, float* scales_dev, int8_t* quants_dev, void* stream) {
    if (!x_dev || !scales_dev || !quants_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (k % QK) return fail(WICK_CUDA_ERR_BAD_ARG, "quantize_q8_0: k must be divisible by 32");
    if (((uintptr_t)x_dev & 15) || ((uintptr_t)quants_dev & 3))
        return fail(WICK_CUDA_ERR_BAD_ARG, "quantize_q8_0: x must be 16-byte aligned and quants 4-byte aligned");
    launch_quant_rows((cudaStream_t)stream, x_dev, (int)n, (int)k, scales_dev, quants_dev);
    OP_END();
}

int32_t wick_cuda_gemv_q8(const wick_cuda_weight* w, const float* xs_dev, const int8_t* xq_dev, float* y_dev, void* stream) {
    if (!w || !xs_dev || !xq_dev || !y_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    GemvJob j{};
    j.count = 1;
    j.w[0] = w->w;
    j.y[0] = y_dev;
    launch_gemv((cudaStream_t)stream, j, xs_dev, xq_dev);
    OP_END();
}

int32_t wick_cuda_gemm_q8(const wick_cuda_weight* w, const float* bs_dev, const int8_t* bq_dev, uint32_t n, float* out_dev,
                          void* stream) {
    if (!w || !bs_dev || !bq_dev || !out_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    launch_gemm((cudaStream_t)stream, w->w, bs_dev, bq_dev, (int)n, out_dev);
    OP_END();
}

// The int8 copy of an operator-API weight, made on first use.
static int32_t ensure_tc_weight(wick_cuda_weight* w, cudaStream_t st) {
    if (w->tc.q) return WICK_CUDA_OK;
    TcWeight t;
    t.m = w->w.m;
    t.k = w->w.k;
    t.m_pad = (w->w.m + 127) / 128 * 128;
    CU_TRY(cudaMalloc((void**)&t.q, t.q_bytes()));
    CU_TRY(cudaMalloc((void**)&t.scales_t, t.s_bytes()));
    CU_TRY(cudaMalloc((void**)&w->tc_err, 4));
    CU_TRY(cudaMemsetAsync(w->tc_err, 0, 4, st));
    w->tc = t;
    CU_TRY(tc_weight_fill(st, w->w, &w->tc));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_gemm_q8_tc(wick_cuda_weight* w, const float* bs_dev, const int8_t* bq_dev, uint32_t n, float* out_dev,
                             int32_t* block_sums_dev, void* stream) {
    if (!w || !bs_dev || !bq_dev || !out_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (!tc_gemm_supported(w->w.m, w->w.k)) return fail(WICK_CUDA_ERR_BAD_ARG, "tensor-core GEMM needs k to be a multiple of 128");
    if (n == 0) return WICK_CUDA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    W_TRY(ensure_tc_weight(w, st));
    CUtensorMap map_x[2];
    CU_TRY(tc_make_activation_map(bq_dev, (int)n, w->w.k, 64, &map_x[0]));
    CU_TRY(tc_make_activation_map(bq_dev, (int)n, w->w.k, 128, &map_x[1]));
    const TcWeight* tw[1] = {&w->tc};
    float* outs[1] = {out_dev};
    CU_TRY(launch_gemm_tc(st, tw, outs, 1, map_x, bs_dev, (int)n, block_sums_dev, w->tc_err));
    uint32_t code = 0;
    CU_TRY(cudaMemcpyAsync(&code, w->tc_err, 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    if (code != 0) {
        cudaMemsetAsync(w->tc_err, 0, 4, st);
        return fail(WICK_CUDA_ERR_TIMEOUT, "tensor-core GEMM: a bounded wait expired (role code " + std::to_string(code) + ")");
    }
    return WICK_CUDA_OK;
}

int32_t wick_cuda_gemm_q8_tc_exact(wick_cuda_weight* w, const float* bs_dev, const int8_t* bq_dev, uint32_t n, float* out_dev,
                                   void* stream) {
    if (!w || !bs_dev || !bq_dev || !out_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (!tc_gemm_supported(w->w.m, w->w.k)) return fail(WICK_CUDA_ERR_BAD_ARG, "tensor-core GEMM needs k to be a multiple of 128");
    if (n == 0) return WICK_CUDA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    W_TRY(ensure_tc_weight(w, st));
    int8_t* xm = nullptr;
    CU_TRY(cudaMalloc((void**)&xm, (size_t)4 * n * w->w.k));
    struct Guard {
        int8_t* p;
        ~Guard() { cudaFree(p); }
    } guard{xm};
    launch_tc_mask_expand(st, bq_dev, (int)n, w->w.k, xm);
    CUtensorMap map_xm;
    CU_TRY(tc_make_activation_map(xm, 4 * (int)n, w->w.k, 64, &map_xm));
    CUtensorMap map_xm32;
    CU_TRY(tc_make_activation_map(xm, 4 * (int)n, w->w.k, 32, &map_xm32));
    const TcWeight* tw[1] = {&w->tc};
    float* outs[1] = {out_dev};
    CU_TRY(launch_gemm_tc_exact(st, tw, outs, 1, map_xm, bs_dev, (int)n, w->tc_err, &map_xm32));
    uint32_t code = 0;
    CU_TRY(cudaMemcpyAsync(&code, w->tc_err, 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    if (code != 0) {
        cudaMemsetAsync(w->tc_err, 0, 4, st);
        return fail(WICK_CUDA_ERR_TIMEOUT, "tensor-core GEMM: a bounded wait expired (role code " + std::to_string(code) + ")");
    }
    return WICK_CUDA_OK;
}

int32_t wick_cuda_block_sums(const wick_cuda_weight* w, const int8_t* xq_dev, int32_t* s_dev, void* stream) {
    if (!w || !xq_dev || !s_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    launch_block_sums((cudaStream_t)stream, w->w, xq_dev, s_dev);
    OP_END();
}

int32_t wick_cuda_rmsnorm(float* x_dev, const float* weight_dev, uint32_t n, uint32_t dim, float eps, void* stream) {
    if (!x_dev || !weight_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (n && dim) launch_rmsnorm((cudaStream_t)stream, x_dev, weight_dev, (int)n, (int)dim, eps);
    OP_END();
}

int32_t wick_cuda_silu_mul(float* gate_dev, const float* up_dev, uint64_t count, void* stream) {
    if (!gate_dev || !up_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    launch_silu_mul((cudaStream_t)stream, gate_dev, up_dev, count);
    OP_END();
}

int32_t wick_cuda_expf(const float* x_dev, float* y_dev, uint64_t count, void* stream) {
    if (!x_dev || !y_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    launch_expf((cudaStream_t)stream, x_dev, y_dev, count);
    OP_END();
}

int32_t wick_cuda_rope(float* q_dev, float* k_dev, uint32_t pos, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                       float freq_base, void* stream) {
    if (!q_dev || !k_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (head_dim % 2 || head_dim > 512) return fail(WICK_CUDA_ERR_BAD_ARG, "head_dim must be even and <= 512");
    const int half = head_dim / 2;
    std::vector<float> tab(2 * half);
    float theta_scale = powf(freq_base, -2.0f / (float)head_dim);
    float theta = (float)pos;
    for (int i = 0; i < half; i++) {
        tab[i] = cosf(theta);
        tab[half + i] = sinf(theta);
        theta *= theta_scale;
    }
    float* dtab = nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    CU_TRY(cudaMallocAsync((void**)&dtab, tab.size() * 4, st));
    CU_TRY(cudaMemcpyAsync(dtab, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, st));
    launch_rope(st, q_dev, k_dev, dtab, dtab + half, (int)n_heads, (int)n_kv_heads, (int)head_dim);
    CU_TRY(cudaStreamSynchronize(st));  // `tab` is pageable host memory
    CU_TRY(cudaFreeAsync(dtab, st));
    OP_END();
}

int32_t wick_cuda_qknorm_rope_kv(float* q_dev, const float* k_dev, const float* v_dev, const float* q_norm_dev, const float* k_norm_dev,
                                 float eps, const float* rope_cos_dev, const float* rope_sin_dev, float* k_cache_dev, float* v_cache_dev,
                                 uint32_t n, uint32_t start_pos, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, void* stream) {
    if (!q_dev || !k_dev || !v_dev || !q_norm_dev || !k_norm_dev || !rope_cos_dev || !rope_sin_dev || !k_cache_dev || !v_cache_dev)
        return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (!n_heads || !n_kv_heads || head_dim % 2 || head_dim > 256 || head_dim == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "bad head shape");
    if (n)
        launch_qknorm_rope_kv((cudaStream_t)stream, q_dev, k_dev, v_dev, q_norm_dev, k_norm_dev, eps, rope_cos_dev, rope_sin_dev, k_cache_dev,
                              v_cache_dev, (int)n, (int)start_pos, nullptr, (int)n_heads, (int)n_kv_heads, (int)head_dim);
    OP_END();
}

int32_t wick_cuda_attention_decode(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev, float* out_dev,
                                   uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t seq, void* stream) {
    return wick_cuda_attention_prefill(q_dev, k_cache_dev, v_cache_dev, out_dev, 1, seq ? seq - 1 : 0, n_heads, n_kv_heads,
                                       head_dim, 0, stream);
}

int32_t wick_cuda_attention_decode_splitk(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev, float* out_dev,
                                          uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t seq, void* stream) {
    if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (!n_kv_heads || n_heads % n_kv_heads || head_dim % 8 || head_dim > 256 || seq == 0) return fail(WICK_CUDA_ERR_BAD_ARG, "bad attention shape");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t floats = attention_splitk_scratch_floats(1, (int)n_heads, (int)head_dim, (int)seq);
    float* scratch = nullptr;
    CU_TRY(cudaMallocAsync((void**)&scratch, floats * 4 + 16, st));
    uint32_t* pos = (uint32_t*)(scratch + floats);
    const uint32_t p = seq - 1;
    CU_TRY(cudaMemcpyAsync(pos, &p, 4, cudaMemcpyHostToDevice, st));
    launch_attention_splitk(st, q_dev, nullptr, nullptr, k_cache_dev, v_cache_dev, pos, out_dev, scratch, 1, (int)n_heads, (int)n_kv_heads,
                            (int)head_dim, (int)seq);
    CU_TRY(cudaStreamSynchronize(st));  // `p` is on this function's stack
    CU_TRY(cudaFreeAsync(scratch, st));
    OP_END();
}

int32_t wick_cuda_attention_prefill(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev, float* out_dev,
                                    uint32_t n, uint32_t start_pos, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                    int32_t flash, void* stream) {
    if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (!n_kv_heads || n_heads % n_kv_heads || head_dim % 8 || head_dim > 256 || n == 0)
        return fail(WICK_CUDA_ERR_BAD_ARG, "bad attention shape");
    if (flash) {
        if (!attention_flash_supported((int)n_heads, (int)n_kv_heads, (int)head_dim))
            return fail(WICK_CUDA_ERR_BAD_ARG, "tiled attention supports head_dim 32, 64 or 128 and at most 8 query heads per KV head");
        cudaStream_t st = (cudaStream_t)stream;
        uint32_t* err = nullptr;
        CU_TRY(cudaMallocAsync((void**)&err, 4, st));
        CU_TRY(cudaMemsetAsync(err, 0, 4, st));
        CU_TRY(launch_attention_flash(st, q_dev, k_cache_dev, v_cache_dev, out_dev, (int)n, (int)start_pos, (int)n_heads, (int)n_kv_heads,
                                      (int)head_dim, err));
        uint32_t code = 0;
        CU_TRY(cudaMemcpyAsync(&code, err, 4, cudaMemcpyDeviceToHost, st));
        CU_TRY(cudaStreamSynchronize(st));
        CU_TRY(cudaFreeAsync(err, st));
        if (code) return fail(WICK_CUDA_ERR_TIMEOUT, "tiled attention: a bounded wait expired (code " + std::to_string(code) + ")");
    } else {
        size_t smem = naive_attention_smem_bytes((int)head_dim, (int)(start_pos + n));
        if (smem > 200 * 1024) return fail(WICK_CUDA_ERR_BAD_ARG, "sequence too long for the per-token attention kernel");
        if (smem > 48 * 1024) {
                configure_naive_attention_smem(smem);
        }
        launch_attention_naive((cudaStream_t)stream, q_dev, k_cache_dev, v_cache_dev, out_dev, (int)n, (int)start_pos, nullptr,
                               (int)n_heads, (int)n_kv_heads, (int)head_dim, (int)(start_pos + n));
    }
    OP_END();
}

int32_t wick_cuda_shortconv(const float* proj_dev, const float* conv_w_dev, float* state_dev, float* out_dev, uint32_t n,
                            uint32_t hidden, uint32_t kernel_size, void* stream) {
    if (!proj_dev || !conv_w_dev || !state_dev || !out_dev) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (hidden % QK || kernel_size < 1 || kernel_size > 8) return fail(WICK_CUDA_ERR_BAD_ARG, "bad short-conv shape");
    launch_shortconv((cudaStream_t)stream, proj_dev, conv_w_dev, state_dev, (int)n, (int)hidden, (int)kernel_size, out_dev, nullptr,
                     nullptr);
    OP_END();
}

int32_t wick_cuda_sample_logits(const float* logits_dev, uint32_t count, float temperature, uint32_t top_k, float top_p, float r,
                                uint32_t* out_dev, void* stream) {
    if (!logits_dev || !out_dev || !count) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument or empty input");
    if (temperature <= 0.0f || top_k == 1) return wick_cuda_argmax(logits_dev, count, out_dev, stream);
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* scratch = nullptr;
    CU_TRY(cudaMallocAsync((void**)&scratch, (size_t)count * 8 + 16, st));
    uint32_t* status = (uint32_t*)(scratch + (size_t)count * 8);
    CU_TRY(cudaMemsetAsync(status, 0, 4, st));
    launch_sample(st, logits_dev, (int)count, temperature, (int)top_k, top_p, r, (float*)scratch, (int*)(scratch + (size_t)count * 4), out_dev, status);
    uint32_t code = 0;
    CU_TRY(cudaMemcpyAsync(&code, status, 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    CU_TRY(cudaFreeAsync(scratch, st));
    if (code) return fail(WICK_CUDA_ERR_BAD_ARG, "on-device top-p needs at most 4096 logits at or above the top-k threshold");
    OP_END();
}

int32_t wick_cuda_argmax(const float* logits_dev, uint32_t count, uint32_t* out_dev, void* stream) {
    if (!logits_dev || !out_dev || !count) return fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument or empty input");
    cudaStream_t st = (cudaStream_t)stream;
    unsigned long long* scratch = nullptr;
    CU_TRY(cudaMallocAsync((void**)&scratch, 8, st));
    CU_TRY(cudaMemsetAsync(scratch, 0, 8, st));
    launch_argmax(st, logits_dev, (int)count, scratch, out_dev);
    CU_TRY(cudaFreeAsync(scratch, st));
    OP_END();
}

}  // extern "C"
