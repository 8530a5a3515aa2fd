// Parameter blocks of the persistent decode kernel (decode_mega.cu).
#pragma once
#include "kernels.cuh"

namespace wick {

// 15 consumer warps + 1 producer warp = 512 threads: the compiler budgets registers for a block size
// rounded up to a multiple of 128, so 17 warps would cap every thread at 96 registers instead of 128.
constexpr int MEGA_CONSUMER_WARPS = 15;
constexpr int MEGA_TEAM_WARPS = 3;
constexpr int MEGA_TEAMS = MEGA_CONSUMER_WARPS / MEGA_TEAM_WARPS;  // the ring has a multiple of this many slots
static_assert(MEGA_CONSUMER_WARPS % MEGA_TEAM_WARPS == 0, "consumer warps must split into whole teams");
constexpr int MEGA_THREADS = 32 * (MEGA_CONSUMER_WARPS + 1);  // warp 0 issues the bulk copies

enum MegaPhaseKind : int {
    MPH_NORM = 0,   // input = RMSNorm(hidden) (first phase of a token: hidden = embedding row)
    MPH_CONV = 1,   // input = c * shortconv(b * x) from proj
    MPH_ATTN = 2,   // no matmul: QK-norm, RoPE, KV append, single-query attention per head
    MPH_QUANT = 3,  // input = a vector produced by the previous phase (attn_out, or the fused SwiGLU output)
    MPH_SILU = 4,   // input = silu(gate) * up, recomputed by every CTA (when the fused form is unavailable)
    MPH_SCORES = 5, // long contexts only, before MPH_ATTN of the same layer: q.k of the cached keys, the keys of every
                    // head split over ALL CTAs, raw scaled scores to global memory (no mat-vec)
};

enum MegaEpilogue : int {
    MEP_STORE = 0,   // y[row] = v
    MEP_ADD = 1,     // y[row] = y[row] + v          (residual add, cpu::add_inplace)
    MEP_LOGITS = 2,  // store (optional) + running argmax
    MEP_SWIGLU = 3,  // paired phase: y[row] = silu(mat[0] row) * (mat[1] row)   (cpu::silu_mul_inplace)
};

struct MegaMat {
    DevWeight w;
    float* y;
    int epi;
};

struct MegaPhase {
    int kind;
    int n_mat;
    int k;              // input length
    int layer;          // conv / attention layer this phase belongs to (or -1)
    int embed;          // MPH_NORM: 1 = first phase of a token
    int conv_commit;    // MPH_NORM: layer whose conv state is advanced in this prologue, or -1
    int pair;           // 1: mat[0] / mat[1] are gate / up of equal shape, streamed as alternating stages and
                        //    combined row by row in the epilogue (MEP_SWIGLU)
    int flag_in;        // MPH_NORM: the hidden row is taken from the flagged copy the previous phase wrote, element by
                        //    element as it arrives; no grid barrier in front of this phase
    int flag_out;       // MEP_ADD phase in front of a flag_in phase: rows are also written as (phase id, value) words
                        //    and the phase does not arrive at the grid barrier (the arrival is made up at the next one)
    const float* src;   // MPH_QUANT: the vector to quantise
    const float* norm_w;
    MegaMat mat[3];
};

struct MegaLayer {
    const float* conv_w;
    float* conv_state;
    const float* q_norm;
    const float* k_norm;
    float* k_cache;
    float* v_cache;
    int n_kv;
};

struct MegaParams {
    const MegaPhase* phases;
    const MegaLayer* layers;
    int n_phases;
    int n_layers;
    int n_tokens;
    int greedy;      // 1: feed the argmax back; 0: single step, logits only
    int hs, is, n_heads, head_dim, vocab, conv_ks, max_seq;
    float eps;
    DevWeight embd;
    // token_embd stored as Q6_K: phase 0 reads its rows from embd6, and the step ends after the last layer
    // (skip_logits): output norm, logits, argmax and the control-block update run as separate kernels
    int embd_q6k, skip_logits;
    DevQ6K embd6;
    float *hidden, *proj, *qbuf, *kbuf, *vbuf, *attn_out, *gate, *up, *logits;
    const float *rope_cos, *rope_sin;
    DecodeCtl* ctl;
    uint32_t* ring;
    int ring_len;
    unsigned long long* hidden_flagged;  // [hs] (phase id << 32 | f32 bits) copy of the hidden row (flag_in / flag_out)
    unsigned long long* bar_counter;   // monotonically increasing arrival counter
    unsigned long long bar_base;       // barriers completed before this launch
    unsigned long long* argmax_acc;    // [2], alternating by token
    int slot_bytes, n_slots;           // bulk-copy ring geometry
    int kmax;                          // max input length over phases (shared-memory sizing)
    int long_ctx;                      // 1: the phase list has MPH_SCORES phases and MPH_ATTN reads the scores they wrote
    float* scores_g;                   // [n_heads][max_seq] scaled scores of the cached keys (long_ctx)
    int uniform_dtype;                 // DT_Q4_0 / DT_Q8_0 when every streamed matrix has that type, else 0
    int xf_extra;                      // extra floats of attention staging (the shared memory left over by the ring)
    // optional per-phase timestamps (globaltimer ns) of CTA 0 for the last step of a launch:
    // [phase][0] barrier passed, [1] prologue done, [2] mat-vec done, [3] arrived
    unsigned long long* prof;          // [n_phases * 4 + 16]
    int prof_phase;                    // phase that also records up to 16 internal stamps after the table
};

// Longest hidden row a flag_in phase handles (15 consumer warps x 5 blocks x 32 elements).
constexpr int MEGA_FLAGGED_MAX_K = 2400;

size_t mega_smem_bytes(const MegaParams& P);
// Launches the persistent kernel (cooperative: one CTA per SM, all co-resident).
cudaError_t launch_decode_mega(cudaStream_t st, const MegaParams& P, int n_ctas);
// Largest grid that is guaranteed co-resident for this configuration on the current device.
int mega_max_ctas(const MegaParams& P);

}  // namespace wick
