// Tensor-parallel all-reduce fused with the step that consumes it, over peer memory on one NVLink / NVSwitch node.
//
// wick has no multi-device path (one sequence, one device).  In a tensor-parallel split of the LFM2 layers every
// row-split mat-vec (attention output, short-conv out_proj, FFN down) leaves each rank with a partial sum of the
// hidden row; the next thing the layer does with the full sum is  hidden += sum; RMSNorm; Q8_0 quantise  (lfm2.rs:
// 1020-1124).  At decode size the message is hidden_size floats (8 KB): far too small for a ring or tree, so this is a
// ONE-SHOT all-reduce: every rank publishes its partial in its own buffer, raises a flag, waits for the flags of
// the others and reads their partials directly with plain loads over NVLink, adding them in rank order (every rank
// adds in the same order, so the replicated hidden rows stay bit-identical across ranks), then runs the residual
// add, the norm and the quantiser in the same kernel.
//
// Buffers are exchanged between the ranks' processes as CUDA IPC handles.  Flags and partials are double-buffered by
// call parity: a rank can only start call n + 2 after it has finished call n + 1, which needed every peer's flag of
// call n + 1, which that peer raised after it had finished reading call n: so a buffer half is never overwritten
// while a peer still reads it.  Every wait is bounded (about a second): on expiry the kernel records a status code
// and returns without touching the outputs, and the context stays usable.  No multicast / multimem is used.
#include <cstring>
#include <string>
#include <vector>

#include "../../include/wick_cuda.h"
#include "common.cuh"

namespace wick {
extern thread_local unsigned long long g_kernel_launches;
}
using namespace wick;

namespace {

constexpr int TP_MAX_WORLD = 8;
constexpr int TP_THREADS = 512;
constexpr unsigned TP_SPIN_LIMIT = 1u << 21;  // x (one system-scope load over NVLink + 200 ns back-off): about a second

struct TpPeers {
    const unsigned int* flags[TP_MAX_WORLD];  // [2] per rank
    const float* data[TP_MAX_WORLD];          // [2][max_floats] per rank
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer4(const float* p) {  // 16-byte aligned
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// One CTA.  `seq` is the 1-based number of this call on the communicator; the half used is seq & 1.
__global__ void __launch_bounds__(TP_THREADS) k_tp_allreduce_add_rmsnorm_quant(TpPeers peers, unsigned int* my_flags, int world, int rank,
                                                                               unsigned int seq, int max_floats, float* __restrict__ hidden,
                                                                               const float* __restrict__ weight, float eps, int dim,
                                                                               float* __restrict__ q8s, int8_t* __restrict__ q8q,
                                                                               float* __restrict__ normed_out, unsigned int* __restrict__ status) {
    extern __shared__ __align__(16) float xs[];
    __shared__ double red[32];
    __shared__ int failed;
    const int half = (int)(seq & 1u);
    if (threadIdx.x == 0) {
        failed = 0;
        // this rank's partial was written by earlier work on this stream: make it visible system-wide, then publish
        __threadfence_system();
        st_release_sys(my_flags + half, seq);
    }
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank) {
        const unsigned int* f = peers.flags[threadIdx.x] + half;
        unsigned spins = 0;
        // (flags only grow; a later call's value on the same half also means this call's data was published, but it
        // cannot appear before this rank has taken part in the call in between)
        while ((int)(ld_acquire_sys(f) - seq) < 0) {
            if (++spins > TP_SPIN_LIMIT) {
                atomicOr(status, 1u << threadIdx.x);
                failed = 1;
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
    if (failed) return;
    // every peer's piece is requested before the first addition, so the loop costs one NVLink round trip, not `world`
    for (int i4 = threadIdx.x; i4 < dim / 4; i4 += blockDim.x) {
        float4 part[TP_MAX_WORLD];
#pragma unroll
        for (int p = 0; p < TP_MAX_WORLD; p++)
            if (p < world) part[p] = ld_peer4(peers.data[p] + (size_t)half * max_floats + 4 * i4);
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < TP_MAX_WORLD; p++)
            if (p < world) {
                sum.x = __fadd_rn(sum.x, part[p].x);
                sum.y = __fadd_rn(sum.y, part[p].y);
                sum.z = __fadd_rn(sum.z, part[p].z);
                sum.w = __fadd_rn(sum.w, part[p].w);
            }
        float4 h = reinterpret_cast<float4*>(hidden)[i4];
        h.x = __fadd_rn(h.x, sum.x);
        h.y = __fadd_rn(h.y, sum.y);
        h.z = __fadd_rn(h.z, sum.z);
        h.w = __fadd_rn(h.w, sum.w);
        reinterpret_cast<float4*>(hidden)[i4] = h;
        reinterpret_cast<float4*>(xs)[i4] = h;
    }
    __syncthreads();
    if (!weight) return;  // plain all-reduce + residual add
    const double sum_sq = block_sum_sq_f64(xs, dim, red);
    const double mean = sum_sq / (double)dim;
    const float inv = (float)(1.0 / sqrt(mean + (double)eps));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int nb = dim / QK;
    for (int b = warp; b < nb; b += nw) {
        const int i = b * QK + lane;
        const float v = __fmul_rn(__fmul_rn(xs[i], inv), weight[i]);
        if (normed_out) normed_out[i] = v;
        if (q8q) {
            float sc;
            const int8_t q = quantize_lane(v, &sc);
            q8q[i] = q;
            if (lane == 0) q8s[b] = sc;
        }
    }
}

thread_local std::string g_tp_error;
int32_t tp_fail(int32_t code, const std::string& msg) {
    g_tp_error = msg;
    return code;
}

}  // namespace

struct wick_cuda_tp_comm {
    int world = 0, rank = 0, device = 0, max_floats = 0;
    unsigned int seq = 0;
    uint8_t* base = nullptr;  // own buffer: [2] flags (padded to 256 bytes), then [2][max_floats] floats
    std::vector<void*> opened;  // peers' mappings
    TpPeers peers{};
    unsigned int* status = nullptr;  // device word: bit p set = gave up waiting for rank p
    bool connected = false;
};

namespace {
size_t tp_bytes(int max_floats) { return 256 + (size_t)2 * max_floats * sizeof(float); }
}

extern "C" {

const char* wick_cuda_tp_last_error(void) { return g_tp_error.c_str(); }

int32_t wick_cuda_tp_comm_create(uint32_t world, uint32_t rank, uint32_t max_floats, wick_cuda_tp_comm** out) {
    if (!out) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "out is NULL");
    *out = nullptr;
    if (world < 1 || world > TP_MAX_WORLD || rank >= world) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "world must be 1..8 and rank < world");
    if (max_floats == 0 || max_floats % QK || max_floats > 12288)
        return tp_fail(WICK_CUDA_ERR_BAD_ARG, "max_floats must be a positive multiple of 32, at most 12288");
    wick_cuda_tp_comm* c = new wick_cuda_tp_comm();
    c->world = (int)world;
    c->rank = (int)rank;
    c->max_floats = (int)max_floats;
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->base, tp_bytes(c->max_floats));
    if (e == cudaSuccess) e = cudaMemset(c->base, 0, tp_bytes(c->max_floats));
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->status, 256);
    if (e == cudaSuccess) e = cudaMemset(c->status, 0, 256);
    if (e != cudaSuccess) {
        cudaFree(c->base);
        cudaFree(c->status);
        delete c;
        return tp_fail(e == cudaErrorMemoryAllocation ? WICK_CUDA_ERR_OOM : WICK_CUDA_ERR_CUDA, std::string("tp_comm_create: ") + cudaGetErrorString(e));
    }
    c->peers.flags[rank] = (const unsigned int*)c->base;
    c->peers.data[rank] = (const float*)(c->base + 256);
    c->connected = world == 1;
    *out = c;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_tp_comm_export(wick_cuda_tp_comm* c, uint8_t* handle_out) {
    if (!c || !handle_out) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == WICK_CUDA_TP_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, c->base);
    if (e != cudaSuccess) return tp_fail(WICK_CUDA_ERR_CUDA, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    memcpy(handle_out, &h, sizeof(h));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_tp_comm_connect(wick_cuda_tp_comm* c, const uint8_t* handles) {
    if (!c || !handles) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (c->connected) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "communicator is already connected");
    cudaError_t e = cudaSetDevice(c->device);
    for (int p = 0; p < c->world && e == cudaSuccess; p++) {
        if (p == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)p * sizeof(h), sizeof(h));
        void* ptr = nullptr;
        e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) break;
        c->opened.push_back(ptr);
        c->peers.flags[p] = (const unsigned int*)ptr;
        c->peers.data[p] = (const float*)((uint8_t*)ptr + 256);
    }
    if (e != cudaSuccess) return tp_fail(WICK_CUDA_ERR_CUDA, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
    c->connected = true;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_tp_partial_buffer(wick_cuda_tp_comm* c, float** partial_dev) {
    if (!c || !partial_dev) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    const unsigned int next = c->seq + 1;
    *partial_dev = (float*)(c->base + 256) + (size_t)(next & 1u) * c->max_floats;
    return WICK_CUDA_OK;
}

int32_t wick_cuda_tp_allreduce_add_rmsnorm_quant(wick_cuda_tp_comm* c, float* hidden_dev, const float* norm_w_dev, float eps, uint32_t dim,
                                                 float* q8s_dev, int8_t* q8q_dev, float* normed_out_dev, void* stream) {
    if (!c || !hidden_dev) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    if (!c->connected) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "communicator is not connected");
    if (dim == 0 || dim % QK || (int)dim > c->max_floats) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "dim must be a multiple of 32 within the communicator's size");
    if ((uintptr_t)hidden_dev & 15) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "hidden_dev must be 16-byte aligned");
    if (norm_w_dev && q8q_dev && !q8s_dev) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "q8s_dev is NULL");
    c->seq += 1;
    g_kernel_launches++;
    k_tp_allreduce_add_rmsnorm_quant<<<1, TP_THREADS, dim * sizeof(float), (cudaStream_t)stream>>>(
        c->peers, (unsigned int*)c->base, c->world, c->rank, c->seq, c->max_floats, hidden_dev, norm_w_dev, eps, (int)dim, q8s_dev, q8q_dev,
        normed_out_dev, c->status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tp_fail(WICK_CUDA_ERR_CUDA, std::string("tp all-reduce launch: ") + cudaGetErrorString(e));
    return WICK_CUDA_OK;
}

int32_t wick_cuda_tp_status(wick_cuda_tp_comm* c, void* stream, uint32_t* gave_up_mask) {
    if (!c || !gave_up_mask) return tp_fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument");
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemcpy(gave_up_mask, c->status, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return tp_fail(WICK_CUDA_ERR_CUDA, std::string("tp_status: ") + cudaGetErrorString(e));
    if (*gave_up_mask) {
        cudaMemset(c->status, 0, 4);
        return tp_fail(WICK_CUDA_ERR_TIMEOUT, "tensor-parallel all-reduce gave up waiting for rank mask " + std::to_string(*gave_up_mask));
    }
    return WICK_CUDA_OK;
}

void wick_cuda_tp_comm_destroy(wick_cuda_tp_comm* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (void* p : c->opened) cudaIpcCloseMemHandle(p);
    cudaFree(c->base);
    cudaFree(c->status);
    delete c;
}

}  // extern "C"
