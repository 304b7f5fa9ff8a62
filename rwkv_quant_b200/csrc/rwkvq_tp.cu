// Tensor-parallel plumbing for the row-split GEMV: symmetric buffers shared between the
// ranks of one node through CUDA IPC, and an all-gather whose data path is plain peer
// stores over NVLink (no library collective, no multicast object, no TMA):
//
//   every rank r holds its slice (count floats) of a vector; rwkvq_tp_allgather_store
//   writes that slice into segment r of the destination buffer of EVERY rank (its own
//   included), makes the stores visible system-wide, raises flag[r] = epoch in every
//   rank's flag array, and then waits until all `world` flags of its own array have
//   reached the epoch (the number of this exchange, counted on the device).  When the
//   kernel completes, the local destination buffer holds the whole vector and later
//   kernels of the stream may read it.
//
// Every wait is bounded: after max_spins polls the kernel stores RWKVQ_E_TIMEOUT in the
// status word and returns, so a rank that never arrives (crashed, or not launched) cannot
// hang the others' GPUs.  A destination buffer may be overwritten by a peer as soon as that
// peer has finished the previous exchange, so callers alternate between two destination
// buffers per exchange site (a rank can be at most one exchange ahead of its peers).
#include "rwkvq_common.cuh"

namespace rwkvq {

constexpr int kTpMaxWorld = 8;

struct TpArgs {
    const float* src;
    float* dst[kTpMaxWorld];            // peer-mapped destination buffers, index = rank
    unsigned int* flags[kTpMaxWorld];   // peer-mapped flag arrays [world]
    int count, rank, world;
    unsigned int* epoch_ctr;            // [world] exchange counters of this rank, one per CTA
    long long max_spins;
    int* status;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// grid = world CTAs: CTA p pushes the slice to rank p, then waits for rank p's slice.
__global__ void __launch_bounds__(256) tp_allgather_store_kernel(const TpArgs a) {
    const int p = blockIdx.x;
    pdl_wait();                                             // the slice comes from the previous kernel
    float* out = a.dst[p] + static_cast<size_t>(a.rank) * a.count;
    const int n4 = a.count >> 2;
    for (int i = threadIdx.x; i < n4; i += blockDim.x)
        reinterpret_cast<float4*>(out)[i] = __ldcg(reinterpret_cast<const float4*>(a.src) + i);
    for (int i = (n4 << 2) + threadIdx.x; i < a.count; i += blockDim.x) out[i] = __ldcg(a.src + i);
    __syncthreads();                // the release below is cumulative over the CTA's stores
    if (threadIdx.x == 0) {
        // the exchange number lives on the device so that a captured graph can be replayed
        const unsigned int epoch = a.epoch_ctr[p] + 1;
        a.epoch_ctr[p] = epoch;
        st_release_sys(a.flags[p] + a.rank, epoch);
        // now wait for rank p's slice in the local buffer
        const unsigned int* mine = a.flags[a.rank] + p;
        long long spins = 0;
        bool ok = true;
        while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
            if (++spins > a.max_spins) { ok = false; break; }
        }
        if (!ok) atomicExch(a.status, RWKVQ_E_TIMEOUT);
        __threadfence_system();
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int rwkvq_tp_alloc(size_t bytes, void** out) {
    RWKVQ_REQUIRE(out != nullptr && bytes > 0, RWKVQ_E_NULL, "rwkvq_tp_alloc: null / empty");
    cudaError_t e = cudaMalloc(out, bytes);
    if (e == cudaSuccess) e = cudaMemset(*out, 0, bytes);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_tp_alloc(%zu): %s", bytes, cudaGetErrorString(e));
    return RWKVQ_OK;
}

int rwkvq_tp_free(void* p) {
    cudaError_t e = cudaFree(p);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_tp_free: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

int rwkvq_ipc_export(const void* dev_ptr, void* handle64) {
    RWKVQ_REQUIRE(dev_ptr && handle64, RWKVQ_E_NULL, "rwkvq_ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr));
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    memcpy(handle64, &h, 64);
    return RWKVQ_OK;
}

int rwkvq_ipc_open(const void* handle64, void** out) {
    RWKVQ_REQUIRE(handle64 && out, RWKVQ_E_NULL, "rwkvq_ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

int rwkvq_ipc_close(void* p) {
    cudaError_t e = cudaIpcCloseMemHandle(p);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

int rwkvq_tp_allgather_store(const float* src, int count, float* const* dst_ptrs, unsigned int* const* flag_ptrs,
                             int rank, int world, unsigned int* epoch_ctr, int* status, long long max_spins, void* stream) {
    RWKVQ_REQUIRE(src && dst_ptrs && flag_ptrs && status && epoch_ctr, RWKVQ_E_NULL, "rwkvq_tp_allgather_store: null pointer");
    RWKVQ_REQUIRE(world >= 1 && world <= kTpMaxWorld && rank >= 0 && rank < world, RWKVQ_E_LIMIT,
                  "rwkvq_tp_allgather_store: rank %d of %d (at most %d ranks)", rank, world, kTpMaxWorld);
    RWKVQ_REQUIRE(count > 0 && aligned(src, 16), RWKVQ_E_ALIGN, "rwkvq_tp_allgather_store: src must be 16-byte aligned");
    RWKVQ_REQUIRE(max_spins > 0, RWKVQ_E_LIMIT, "rwkvq_tp_allgather_store: max_spins must be positive");
    TpArgs a{};
    a.src = src; a.count = count; a.rank = rank; a.world = world; a.epoch_ctr = epoch_ctr; a.max_spins = max_spins;
    a.status = status;
    for (int r = 0; r < world; ++r) {
        RWKVQ_REQUIRE(dst_ptrs[r] && flag_ptrs[r], RWKVQ_E_NULL, "rwkvq_tp_allgather_store: rank %d buffers missing", r);
        RWKVQ_REQUIRE(aligned(dst_ptrs[r], 16) && (count % 4 == 0 || world == 1), RWKVQ_E_ALIGN,
                      "rwkvq_tp_allgather_store: 16-byte aligned buffers and count %% 4 == 0 required");
        a.dst[r] = dst_ptrs[r]; a.flags[r] = flag_ptrs[r];
    }
    cudaError_t e = launch_pdl(tp_allgather_store_kernel, dim3(world), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_tp_allgather_store: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

}  // extern "C"
