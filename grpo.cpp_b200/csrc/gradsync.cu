// Gradient all-reduce fused with the 1/world scale, over NVLink peer memory.
//
// The reference's two-GPU GPT-2 demo sums the replicas' gradients with ncclAllReduce in place and
// then runs scale_kernel over all of them again (apps/05_two_gpu_gpt2_grpo.cu:216-219, 260-268): a
// collective plus a second full read and write of the 124 M floats.  Here ONE kernel per rank does
// both: rank r owns slice r of the buffer; it loads that slice from every rank's buffer (its own
// locally, the others' over NVLink), adds the terms in rank order -- so every replica ends up with
// the same bits, which the demo checks by hashing the replicas (:330-342) --, multiplies by the
// scale, and stores the result into slice r of every rank's buffer.  No library collective, no
// multicast object: plain peer loads and stores.
//
// Synchronisation between the ranks' kernels (each on its own GPU) goes through a small flag block
// per rank: a rank announces "my gradients are final" to everyone when its kernel starts, every
// CTA waits for all announcements before it reads, and the CTA that finishes last on a rank
// announces "my stores into your buffer are done" and waits for the others' announcements, so that
// the kernel's end means this rank's buffer is complete.  Every wait is bounded and ends in an
// error word the host can read.
#include <atomic>
#include <cstring>
#include <new>

#include "common.cuh"

using namespace grpo_b200;

namespace {

constexpr int kMaxWorld = 8;
constexpr int kSyncThreads = 512;
constexpr int kUnroll = 4;  // float4 per thread per step

struct SyncFlags {                                 // one per rank, in device memory every rank maps
    unsigned long long arrived[kMaxWorld];        // [source rank]: the epoch of its last "gradients final"
    unsigned long long finished[kMaxWorld];       // [source rank]: the epoch of its last "stores done"
    unsigned int ticket;                           // CTAs of this rank that finished their slice
    int error;                                     // 1: a wait for a peer gave up
};

struct SyncArgs {
    float* bufs[kMaxWorld];       // every rank's gradient buffer as reachable from this rank
    SyncFlags* flags[kMaxWorld];  // every rank's flag block
    int rank, world;
    long long n;                  // floats
    float scale;
    unsigned long long epoch;
    long long timeout_cycles;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// system-scope accesses: the data was written by (and goes to) other GPUs
__device__ __forceinline__ float4 ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer(float4* p, float4 v) {
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// waits until every rank's word in `words` shows `epoch`; false when the limit ran out
__device__ __forceinline__ bool wait_all(const unsigned long long* words, int world, unsigned long long epoch, long long limit) {
    const long long start = clock64();
    for (int q = 0; q < world; q++) {
        while (ld_acquire_sys(words + q) < epoch) {
            if (clock64() - start > limit) return false;
            __nanosleep(64);
        }
    }
    return true;
}

template <int WORLD>
__global__ void __launch_bounds__(kSyncThreads) allreduce_scale_kernel(const SyncArgs a) {
    __shared__ int go;
    const int tid = threadIdx.x;
    SyncFlags* mine = a.flags[a.rank];
    // "my gradients are final": stream order put this kernel behind whatever produced them
    if (blockIdx.x == 0 && tid < WORLD) st_release_sys(&a.flags[tid]->arrived[a.rank], a.epoch);
    if (tid == 0) {
        go = wait_all(mine->arrived, WORLD, a.epoch, a.timeout_cycles) ? 1 : 0;
        if (!go) atomicExch(&mine->error, 1);
    }
    __syncthreads();
    if (go) {
        // slice r in units of float4; the last rank also takes the floats past the last whole float4
        const long long n4 = a.n >> 2;
        const long long per = (n4 + WORLD - 1) / WORLD;
        const long long first = min(static_cast<long long>(a.rank) * per, n4);
        const long long count = min(first + per, n4) - first;
        // consecutive lanes take consecutive float4s (every load and store instruction of a warp covers 512
        // contiguous bytes); a thread's kUnroll elements lie a whole grid apart
        const long long lanes = static_cast<long long>(gridDim.x) * kSyncThreads;
        for (long long i0 = static_cast<long long>(blockIdx.x) * kSyncThreads + tid; i0 < count; i0 += lanes * kUnroll) {
            float4 acc[kUnroll];
            float4 term[kUnroll][WORLD];
#pragma unroll
            for (int u = 0; u < kUnroll; u++)
#pragma unroll
                for (int q = 0; q < WORLD; q++)
                    if (i0 + u * lanes < count) term[u][q] = ld_peer(reinterpret_cast<const float4*>(a.bufs[q]) + first + i0 + u * lanes);
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                if (i0 + u * lanes >= count) continue;
                acc[u] = term[u][0];
#pragma unroll
                for (int q = 1; q < WORLD; q++) {  // rank order: the same bits on every replica
                    acc[u].x = __fadd_rn(acc[u].x, term[u][q].x);
                    acc[u].y = __fadd_rn(acc[u].y, term[u][q].y);
                    acc[u].z = __fadd_rn(acc[u].z, term[u][q].z);
                    acc[u].w = __fadd_rn(acc[u].w, term[u][q].w);
                }
                acc[u].x = __fmul_rn(acc[u].x, a.scale);
                acc[u].y = __fmul_rn(acc[u].y, a.scale);
                acc[u].z = __fmul_rn(acc[u].z, a.scale);
                acc[u].w = __fmul_rn(acc[u].w, a.scale);
#pragma unroll
                for (int q = 0; q < WORLD; q++) st_peer(reinterpret_cast<float4*>(a.bufs[q]) + first + i0 + u * lanes, acc[u]);
            }
        }
        if (a.rank == WORLD - 1) {  // the up-to-three floats past the last whole float4
            const long long tail = a.n - (n4 << 2);
            const long long g = static_cast<long long>(blockIdx.x) * kSyncThreads + tid;
            if (g < tail) {
                const long long at = (n4 << 2) + g;
                float s = 0.0f;
                for (int q = 0; q < WORLD; q++) {
                    float v;
                    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(a.bufs[q] + at) : "memory");
                    s = q == 0 ? v : __fadd_rn(s, v);
                }
                s = __fmul_rn(s, a.scale);
                for (int q = 0; q < WORLD; q++) asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(a.bufs[q] + at), "f"(s) : "memory");
            }
        }
    }
    // ---- "my stores into your buffers are done", by the CTA that finishes last on this rank
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const bool last = atomicAdd(&mine->ticket, 1u) == gridDim.x - 1;
        if (last) {
            mine->ticket = 0u;  // left as it was found
            __threadfence_system();
            for (int q = 0; q < WORLD; q++) st_release_sys(&a.flags[q]->finished[a.rank], a.epoch);
            if (!wait_all(mine->finished, WORLD, a.epoch, a.timeout_cycles)) atomicExch(&mine->error, 1);
        }
    }
}

}  // namespace

struct grpo_b200_gradsync {
    int device = -1;
    int rank = 0, world = 1;
    float* grads = nullptr;
    long long n = 0;
    void* base = nullptr;    // the allocation that holds grads (what an IPC handle names)
    size_t offset = 0;
    SyncFlags* flags = nullptr;
    float* bufs[kMaxWorld] = {};
    SyncFlags* peer_flags[kMaxWorld] = {};
    void* opened[2 * kMaxWorld] = {};
    int n_opened = 0;
    bool connected = false;
    unsigned long long epoch = 0;
    int sms = 148;
};

namespace {

int bad(const char* msg) {
    set_error("%s", msg);
    return GRPO_B200_E_INVALID;
}

struct Guard {
    int previous = -1;
    explicit Guard(int device) {
        if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
        if (previous != device) cudaSetDevice(device);
    }
    ~Guard() {
        if (previous >= 0) cudaSetDevice(previous);
    }
};

// the allocation an interior device pointer belongs to (cuMemGetAddressRange, reached through the
// runtime so that the library does not link the driver)
cudaError_t allocation_of(const void* p, void** base, size_t* size) {
    using Fn = int (*)(unsigned long long*, size_t*, unsigned long long);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    cudaError_t err = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &status);
    if (err != cudaSuccess) return err;
    if (!fn || status != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
    unsigned long long b = 0;
    size_t s = 0;
    if (reinterpret_cast<Fn>(fn)(&b, &s, reinterpret_cast<unsigned long long>(p)) != 0) return cudaErrorInvalidValue;
    *base = reinterpret_cast<void*>(b);
    *size = s;
    return cudaSuccess;
}

std::atomic<long long> g_sync_timeout{1LL << 33};  // about four seconds

}  // namespace

extern "C" {

void grpo_b200_gradsync_slice(int64_t n, int world, int rank, int64_t* first, int64_t* count) {
    const int64_t n4 = n >> 2;
    const int64_t per = (n4 + world - 1) / world;
    int64_t lo = rank * per < n4 ? rank * per : n4;
    int64_t hi = lo + per < n4 ? lo + per : n4;
    *first = lo * 4;
    *count = (hi - lo) * 4 + (rank == world - 1 ? n - n4 * 4 : 0);
}

int grpo_b200_gradsync_create(int rank, int world, float* grads, int64_t n, grpo_b200_gradsync_t* out) {
    if (!out) return bad("out must not be null");
    *out = nullptr;
    if (world < 1 || world > kMaxWorld) return bad("world must lie in [1, 8]");
    if (rank < 0 || rank >= world) return bad("rank must lie in [0, world)");
    if (!grads || n <= 0) return bad("grads must not be null and n must be positive");
    if (reinterpret_cast<uintptr_t>(grads) & 15u) return bad("grads must be 16-byte aligned");
    grpo_b200_gradsync* h = new (std::nothrow) grpo_b200_gradsync();
    if (!h) return bad("out of host memory");
    h->rank = rank;
    h->world = world;
    h->grads = grads;
    h->n = n;
    cudaError_t err = cudaGetDevice(&h->device);
    size_t size = 0;
    if (err == cudaSuccess) err = allocation_of(grads, &h->base, &size);
    if (err == cudaSuccess) h->offset = static_cast<size_t>(reinterpret_cast<char*>(grads) - static_cast<char*>(h->base));
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->flags), sizeof(SyncFlags));
    if (err == cudaSuccess) err = cudaMemset(h->flags, 0, sizeof(SyncFlags));
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&h->sms, cudaDevAttrMultiProcessorCount, h->device);
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        const int rc = cuda_fail(err, "setting up the gradient exchange");
        grpo_b200_gradsync_destroy(h);
        return rc;
    }
    h->bufs[rank] = grads;
    h->peer_flags[rank] = h->flags;
    h->connected = world == 1;
    *out = h;
    return GRPO_B200_OK;
}

int grpo_b200_gradsync_export(grpo_b200_gradsync_t h, unsigned char handle[192]) {
    static_assert(2 * sizeof(cudaIpcMemHandle_t) + sizeof(unsigned long long) <= 192, "the handle block holds two IPC handles and an offset");
    if (!h || !handle) return bad("handle must not be null");
    Guard guard(h->device);
    cudaIpcMemHandle_t buf, flg;
    GRPO_CUDA_TRY(cudaIpcGetMemHandle(&buf, h->base));
    GRPO_CUDA_TRY(cudaIpcGetMemHandle(&flg, h->flags));
    memset(handle, 0, 192);
    memcpy(handle, &buf, 64);
    memcpy(handle + 64, &flg, 64);
    const unsigned long long off = h->offset;
    memcpy(handle + 128, &off, 8);
    return GRPO_B200_OK;
}

int grpo_b200_gradsync_connect_ipc(grpo_b200_gradsync_t h, const unsigned char* handles) {
    if (!h || !handles) return bad("handles must not be null");
    Guard guard(h->device);
    for (int r = 0; r < h->world; r++) {
        if (r == h->rank || h->bufs[r]) continue;
        const unsigned char* blob = handles + 192 * static_cast<size_t>(r);
        cudaIpcMemHandle_t buf, flg;
        unsigned long long off = 0;
        memcpy(&buf, blob, 64);
        memcpy(&flg, blob + 64, 64);
        memcpy(&off, blob + 128, 8);
        void* pb = nullptr;
        void* pf = nullptr;
        GRPO_CUDA_TRY(cudaIpcOpenMemHandle(&pb, buf, cudaIpcMemLazyEnablePeerAccess));
        h->opened[h->n_opened++] = pb;
        GRPO_CUDA_TRY(cudaIpcOpenMemHandle(&pf, flg, cudaIpcMemLazyEnablePeerAccess));
        h->opened[h->n_opened++] = pf;
        h->bufs[r] = reinterpret_cast<float*>(static_cast<char*>(pb) + off);
        h->peer_flags[r] = static_cast<SyncFlags*>(pf);
    }
    h->connected = true;
    return GRPO_B200_OK;
}

int grpo_b200_gradsync_connect_local(grpo_b200_gradsync_t h, grpo_b200_gradsync_t const* all) {
    if (!h || !all) return bad("the list of handles must not be null");
    Guard guard(h->device);
    for (int r = 0; r < h->world; r++) {
        if (r == h->rank) continue;
        const grpo_b200_gradsync* peer = all[r];
        if (!peer || peer->rank != r || peer->world != h->world || peer->n != h->n)
            return bad("the list must hold every rank's handle for buffers of the same size, in rank order");
        if (peer->device != h->device) {
            int can = 0;
            GRPO_CUDA_TRY(cudaDeviceCanAccessPeer(&can, h->device, peer->device));
            if (!can) return bad("this rank's device cannot reach a peer's memory");
            const cudaError_t err = cudaDeviceEnablePeerAccess(peer->device, 0);
            if (err != cudaSuccess && err != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(err, "enabling peer access");
            if (err == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        }
        h->bufs[r] = peer->grads;
        h->peer_flags[r] = peer->flags;
    }
    h->connected = true;
    return GRPO_B200_OK;
}

int grpo_b200_gradsync_set_timeout_cycles(int64_t cycles) {
    if (cycles <= 0) return bad("the timeout must be a positive number of SM clock cycles");
    g_sync_timeout.store(cycles, std::memory_order_relaxed);
    return GRPO_B200_OK;
}

int grpo_b200_allreduce_scale(grpo_b200_gradsync_t h, float scale, grpo_b200_stream_t stream) {
    if (!h) return bad("handle must not be null");
    if (!h->connected) return bad("the handle is not connected to the other ranks' buffers");
    int current = -1;
    GRPO_CUDA_TRY(cudaGetDevice(&current));
    if (current != h->device) return bad("the handle belongs to another device than the current one");
    SyncArgs a = {};
    for (int r = 0; r < h->world; r++) {
        a.bufs[r] = h->bufs[r];
        a.flags[r] = h->peer_flags[r];
    }
    a.rank = h->rank;
    a.world = h->world;
    a.n = h->n;
    a.scale = scale;
    a.epoch = ++h->epoch;
    a.timeout_cycles = g_sync_timeout.load(std::memory_order_relaxed);
    const long long n4 = h->n >> 2;
    const long long per = (n4 + h->world - 1) / h->world;
    long long blocks = (per + kSyncThreads * kUnroll - 1) / (kSyncThreads * kUnroll);
    const long long cap = static_cast<long long>(h->sms) * 2;  // (no CTA waits for another CTA: the grid need not be resident at once)  // (no CTA waits for another: the grid need not be resident at once)
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>(blocks);
    switch (h->world) {
        case 1: allreduce_scale_kernel<1><<<grid, kSyncThreads, 0, s>>>(a); break;
        case 2: allreduce_scale_kernel<2><<<grid, kSyncThreads, 0, s>>>(a); break;
        case 3: allreduce_scale_kernel<3><<<grid, kSyncThreads, 0, s>>>(a); break;
        case 4: allreduce_scale_kernel<4><<<grid, kSyncThreads, 0, s>>>(a); break;
        case 5: allreduce_scale_kernel<5><<<grid, kSyncThreads, 0, s>>>(a); break;
        case 6: allreduce_scale_kernel<6><<<grid, kSyncThreads, 0, s>>>(a); break;
        case 7: allreduce_scale_kernel<7><<<grid, kSyncThreads, 0, s>>>(a); break;
        default: allreduce_scale_kernel<8><<<grid, kSyncThreads, 0, s>>>(a); break;
    }
    GRPO_CUDA_TRY(cudaGetLastError());
    return GRPO_B200_OK;
}

int grpo_b200_gradsync_status(grpo_b200_gradsync_t h, int* timed_out) {
    if (!h || !timed_out) return bad("handle and timed_out must not be null");
    Guard guard(h->device);
    int err = 0;
    GRPO_CUDA_TRY(cudaMemcpy(&err, &h->flags->error, sizeof(int), cudaMemcpyDeviceToHost));
    *timed_out = err;
    return GRPO_B200_OK;
}

int grpo_b200_gradsync_destroy(grpo_b200_gradsync_t h) {
    if (!h) return GRPO_B200_OK;
    if (h->device >= 0) {
        Guard guard(h->device);
        cudaDeviceSynchronize();
        for (int i = 0; i < h->n_opened; i++)
            if (h->opened[i]) cudaIpcCloseMemHandle(h->opened[i]);
        if (h->flags) cudaFree(h->flags);
    }
    delete h;
    return GRPO_B200_OK;
}

}  // extern "C"
