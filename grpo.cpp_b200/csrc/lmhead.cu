// LM-head projection fused with the loss statistics: logits = hidden x W^T are formed tile by tile on
// the tensor cores and reduced on the spot to what the loss needs per row -- the maximum, the
// normaliser and the selected logit -- so the [N][P] logits are never written to memory.
//
// The reference materialises them: gpt2_forward leaves N x P fp32 logits in model.acts.output and the
// loss boundary then reads them (apps/04_gpt2_grpo.cu:322-331).  This is the forward half of that
// fusion (loss, pg, kl and log p(selected); the backward half would recompute the tiles).
//
// Arithmetic: TF32 inputs (fp32 words whose low 13 mantissa bits the tensor core ignores), fp32
// accumulation -- the precision of the cuBLAS TF32 matmul llm.c runs this projection with, not
// narrower.  A tile unit is 128 rows by 256 vocabulary columns; per CTA:
//   warp 0     TMA producer: per k-block of 32 floats, the 128 x 32 tile of hidden and the 256 x 32 tile
//              of W into a 4-stage ring (cp.async.bulk.tensor, 128-byte swizzle, no multicast);
//   warp 1     issues tcgen05.mma (M=128, N=256, K=8, kind::tf32), accumulators in tensor memory,
//              two buffers of 256 columns so that a tile's epilogue overlaps the next tile's MMAs;
//   warps 2-5  epilogue: tcgen05.ld of the accumulators (one row per thread), running maximum and
//              sum of exponentials, the selected logit when its column passes by.
// The (row block, vocabulary tile) units are cut into equal contiguous shares, one per SM, so a row block's
// vocabulary is covered by several CTAs (and a CTA may finish one row block and start the next); a small
// kernel merges the shares into the row records the reduce kernel of the logits path consumes.
// Every mbarrier wait is bounded; a wait that runs out raises the status word and the CTA winds down.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace grpo_b200 {
namespace {

constexpr int kBM = 128;        // rows per CTA
constexpr int kBN = 256;        // vocabulary columns per tile
constexpr int kBK = 32;         // floats per k-block: 128 bytes, one swizzle row
constexpr int kUmmaK = 8;       // floats per tcgen05.mma of kind::tf32
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr uint32_t kABytes = kBM * kBK * 4;  // 16 KB
constexpr uint32_t kBBytes = kBN * kBK * 4;  // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024;  // + room to align to 1 KB
constexpr int kTmemCols = 512;
#define kNegInfF (-CUDART_INF_F)
constexpr float kLog2eF = 1.4426950408889634f;
constexpr long long kWaitLimit = 1LL << 31;  // about a second of SM clock

struct LmHeadArgs {
    long long n_rows;
    int V, P, C;
    int n_mtiles, n_tiles, n_ctas, max_slots;  // work = n_mtiles * n_tiles tile units, cut evenly over n_ctas CTAs
    const int32_t* selected;
    const int32_t* mask;
    float4* partials;  // [max_slots][n_mtiles * 128]: {max, sum relative to max, selected logit, has selected}
    int* status;
};

// The tile units (row block m, vocabulary tile t) are numbered m * n_tiles + t and cut into n_ctas contiguous
// ranges of nearly equal length; a range may end one row block and start the next.  A row block's partial
// results are numbered by the order of the CTAs that work on it ("slots").
__host__ __device__ inline long long unit_begin(int cta, long long total, int n_ctas) { return total * cta / n_ctas; }
__host__ __device__ inline int cta_of_unit(long long unit, long long total, int n_ctas) {
    int c = static_cast<int>((unit * n_ctas) / total);  // a first guess that is at most one off
    while (c + 1 < n_ctas && unit_begin(c + 1, total, n_ctas) <= unit) c++;
    while (c > 0 && unit_begin(c, total, n_ctas) > unit) c--;
    return c;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded: false when the limit ran out
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    const long long start = clock64();
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) return true;
        if (clock64() - start > kWaitLimit) return false;
    }
}

// 2-D tiled bulk tensor load into this CTA's shared memory (no multicast)
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled:
// groups of 8 rows lie 1024 bytes apart (stride byte offset 64 in 16-byte units); version 1, layout 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>(1) << 16;   // leading byte offset (unused by swizzled K-major layouts)
    d |= static_cast<uint64_t>(64) << 32;  // stride byte offset: 1024 bytes
    d |= static_cast<uint64_t>(1) << 46;   // descriptor version of this architecture
    d |= static_cast<uint64_t>(2) << 61;   // 128-byte swizzle
    return d;
}

// Instruction descriptor: D fp32, A and B tf32, both K-major, N = 256, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(kBN >> 3) << 17) |
                                (static_cast<uint32_t>(kBM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's row (lane of tensor memory)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

__global__ void __launch_bounds__(kThreads, 1)
    lmhead_stats_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const LmHeadArgs a) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full_bar[kStages];
    __shared__ uint64_t empty_bar[kStages];
    __shared__ uint64_t acc_full[2];
    __shared__ uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const long long total_units = static_cast<long long>(a.n_mtiles) * a.n_tiles;
    const long long u0 = unit_begin(blockIdx.x, total_units, a.n_ctas);
    const long long u1 = unit_begin(blockIdx.x + 1, total_units, a.n_ctas);
    const int k_blocks = a.C / kBK;

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            bar_init(&full_bar[s], 1);
            bar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; i++) {
            bar_init(&acc_full[i], 1);
            bar_init(&acc_empty[i], 4);  // one arrival per epilogue warp
        }
        abort_sh = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // one warp allocates the tensor memory (and frees it at the end)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sh;

    if (warp == 0) {
        // ---- producer
        if (lane == 0) {
            unsigned it = 0;
            for (long long u = u0; u < u1 && abort_sh == 0; u++) {
                const int m_tile = static_cast<int>(u / a.n_tiles), t = static_cast<int>(u % a.n_tiles);
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const unsigned s = it % kStages;
                    if (!bar_wait(&empty_bar[s], ((it / kStages) & 1u) ^ 1u)) {
                        atomicExch(&abort_sh, 1);
                        break;
                    }
                    unsigned char* stage = smem + static_cast<size_t>(s) * kStageBytes;
                    bar_expect_tx(&full_bar[s], kStageBytes);
                    tma_load_2d(stage, &map_a, kb * kBK, m_tile * kBM, &full_bar[s]);
                    tma_load_2d(stage + kABytes, &map_b, kb * kBK, t * kBN, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            unsigned it = 0;
            int n_done = 0;
            for (long long u = u0; u < u1 && abort_sh == 0; u++, n_done++) {
                const unsigned ab = n_done & 1u;
                if (!bar_wait(&acc_empty[ab], ((n_done >> 1) & 1u) ^ 1u)) {
                    atomicExch(&abort_sh, 1);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + ab * kBN;
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const unsigned s = it % kStages;
                    if (!bar_wait(&full_bar[s], (it / kStages) & 1u)) {
                        atomicExch(&abort_sh, 1);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + static_cast<size_t>(s) * kStageBytes);
                    const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; k++)  // 32 bytes further along K inside the swizzled row: +2 in the address field
                        umma_tf32(tmem_d, da + 2u * k, db + 2u * k, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
                }
                if (abort_sh != 0) break;
                umma_commit(&acc_full[ab]);  // the tile's accumulators are complete
            }
        }
    } else {
        // ---- epilogue: thread <-> row (lane of tensor memory); a warp reaches lanes 32 * (warp % 4) ...
        const int quarter = warp & 3;
        int m_tile = -1, sel = -1;
        float m_run = kNegInfF, s_run = 0.0f, x_sel = 0.0f, has_sel = 0.0f;
        // this CTA's partial of row block m goes to the slot numbered by the CTAs that work on that block
        auto flush = [&](int m) {
            const int slot = blockIdx.x - cta_of_unit(static_cast<long long>(m) * a.n_tiles, total_units, a.n_ctas);
            const size_t at = (static_cast<size_t>(slot) * a.n_mtiles + m) * kBM + quarter * 32 + lane;
            a.partials[at] = make_float4(m_run, s_run, x_sel, has_sel);
        };
        int n_done = 0;
        for (long long u = u0; u < u1; u++, n_done++) {
            const int m_now = static_cast<int>(u / a.n_tiles), t = static_cast<int>(u % a.n_tiles);
            if (m_now != m_tile) {  // a new row block: hand over the finished one, start afresh
                if (m_tile >= 0) flush(m_tile);
                m_tile = m_now;
                const long long row = static_cast<long long>(m_tile) * kBM + quarter * 32 + lane;
                sel = (row < a.n_rows && a.mask[row] != 0) ? a.selected[row] : -1;
                m_run = kNegInfF;
                s_run = x_sel = has_sel = 0.0f;
            }
            const unsigned ab = n_done & 1u;
            bool ok = abort_sh == 0;
            if (ok) ok = bar_wait(&acc_full[ab], (n_done >> 1) & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                atomicExch(&abort_sh, 1);
                break;
            }
            tc_fence_after();
            const int col0 = t * kBN;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; c++) {
                float v[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + ab * kBN + c * 32, v);
                const int base = col0 + c * 32;
                float cm = kNegInfF;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    if (base + j >= a.V) v[j] = kNegInfF;  // padding columns of the vocabulary (and of the last tile)
                    if (base + j == sel) {
                        x_sel = v[j];
                        has_sel = 1.0f;
                    }
                    cm = fmaxf(cm, v[j]);
                }
                if (cm > m_run) {  // (cm == -inf only for chunks that hold no vocabulary column)
                    s_run *= exp2f((m_run - cm) * kLog2eF);
                    m_run = cm;
                }
                if (m_run != kNegInfF) {
                    const float shift = m_run * kLog2eF;
                    float acc = 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; j++) acc += exp2f(fmaf(v[j], kLog2eF, -shift));
                    s_run += acc;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) bar_arrive(&acc_empty[ab]);  // the buffer may be overwritten by the tile after next
        }
        if (m_tile >= 0) flush(m_tile);
    }

    // ---- wind down: nothing of this CTA is still in flight, then the tensor memory goes back
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && abort_sh != 0) atomicOr(a.status, kStatusPipelineTimeout);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}


// Merges the vocabulary splits of every row into the record the reduce kernel consumes: the row maximum,
// the normaliser relative to it (in double) and the selected logit; a missing selected logit (an id outside
// the vocabulary) is flagged as a bad input.  Also clears the pass's control words for the reduce kernel.
__global__ void __launch_bounds__(256) lmhead_merge_kernel(const float4* __restrict__ partials, int n_mtiles, int n_tiles,
                                                           int n_ctas, LogitsArgs a, double* lse_out) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.counter = 0u;  // (the status word was cleared before the first kernel)
    const long long row = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (row >= a.n_rows) return;
    const bool active = a.mask[row] != 0;
    // the CTAs that worked on this row's block, first to last: as many slots hold a partial
    const long long total_units = static_cast<long long>(n_mtiles) * n_tiles, padded_rows = static_cast<long long>(n_mtiles) * kBM;
    const int m_tile = static_cast<int>(row / kBM);
    const int n_splits = cta_of_unit(static_cast<long long>(m_tile + 1) * n_tiles - 1, total_units, n_ctas) -
                         cta_of_unit(static_cast<long long>(m_tile) * n_tiles, total_units, n_ctas) + 1;
    float m = kNegInfF;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, partials[static_cast<size_t>(s) * padded_rows + row].x);
    double z = 0.0;
    float x_sel = 0.0f, has = 0.0f;
    for (int s = 0; s < n_splits; s++) {
        const float4 p = partials[static_cast<size_t>(s) * padded_rows + row];
        if (p.x != kNegInfF) z += static_cast<double>(p.y) * exp2(static_cast<double>(p.x - m) * 1.4426950408889634);
        if (p.w != 0.0f) {
            x_sel = p.z;
            has = 1.0f;
        }
    }
    RowRecord r;
    r.z = z;
    r.m = m;
    r.x_sel = x_sel;
    r.flags = (active && has == 0.0f) ? kRowBadInput : 0.0f;
    r.pad[0] = r.pad[1] = r.pad[2] = 0.0f;
    a.rows[row] = r;
    if (lse_out) lse_out[row] = active ? static_cast<double>(m) + log(z) : 0.0;
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, reached through the runtime so that the library does not link the driver
cudaError_t encode_fn(EncodeTiled* out) {
    static std::mutex mutex;
    static EncodeTiled cached = nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if (!cached) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        const cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
        if (err != cudaSuccess) return err;
        if (!fn || status != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        cached = reinterpret_cast<EncodeTiled>(fn);
    }
    *out = cached;
    return cudaSuccess;
}

// [rows][C] fp32, row-major; boxes of 32 floats (128 bytes) by box_rows rows, 128-byte swizzle, zeros out of bounds
cudaError_t make_map(EncodeTiled encode, CUtensorMap* map, const float* base, long long rows, int C, int box_rows) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(C) * sizeof(float)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

struct LmHeadPlan {
    int n_mtiles, n_tiles, n_ctas, max_slots;
    long long padded_rows;
};

LmHeadPlan plan_for(long long n_rows, int P, int sms) {
    LmHeadPlan p;
    p.n_mtiles = static_cast<int>((n_rows + kBM - 1) / kBM);
    p.n_tiles = (P + kBN - 1) / kBN;
    const long long total = static_cast<long long>(p.n_mtiles) * p.n_tiles;
    p.n_ctas = static_cast<int>(total < sms ? total : sms);  // one CTA per SM, every SM busy, equal shares of the tiles
    // a row block's tiles are shared by at most this many consecutive CTAs
    const long long shortest = total / p.n_ctas;
    p.max_slots = static_cast<int>((p.n_tiles + shortest - 1) / shortest) + 1;
    p.padded_rows = static_cast<long long>(p.n_mtiles) * kBM;
    return p;
}

int device_sms() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
    return sms;
}

}  // namespace
}  // namespace grpo_b200

using namespace grpo_b200;

extern "C" {

size_t grpo_b200_lmhead_workspace_bytes(int64_t n_rows, int P) {
    if (n_rows <= 0 || P <= 0) return 0;
    const LmHeadPlan p = plan_for(n_rows, P, device_sms());
    // the logits path's workspace (row records, control words, reduce partials), then the split partials
    const size_t base = (grpo_b200_logits_workspace_bytes(n_rows) + 255) & ~static_cast<size_t>(255);
    return base + static_cast<size_t>(p.max_slots) * static_cast<size_t>(p.padded_rows) * sizeof(float4);
}

int grpo_b200_lmhead_loss(const float* hidden, const float* lm_head, int64_t n_rows, int C, int V, int P,
                          const float* logp_old, const float* logp_ref, const int32_t* selected, const float* advantages,
                          const float* weights, const int32_t* mask, int64_t row_offset, int tokens_per_seq,
                          float clip_eps, float beta, float* selected_logp, double* lse_out, grpo_b200_result_t* result,
                          void* workspace, size_t workspace_bytes, grpo_b200_stream_t stream) {
    auto invalid = [](const char* msg) {
        set_error("%s", msg);
        return static_cast<int>(GRPO_B200_E_INVALID);
    };
    if (!hidden || !lm_head) return invalid("hidden and lm_head must not be null");
    if (!logp_old || !logp_ref || !selected || !advantages || !weights || !mask || !result)
        return invalid("device pointers must not be null");
    if (n_rows <= 0 || tokens_per_seq <= 0 || row_offset < 0) return invalid("B, G and T must be positive");
    if (row_offset + n_rows > 2147483647LL) return invalid("token count exceeds INT_MAX");
    if (V <= 0) return invalid("V must be positive");
    if (P < V) return invalid("P must be at least V");
    if (C <= 0 || C % kBK != 0) return invalid("the hidden width must be a positive multiple of 32");
    if ((reinterpret_cast<uintptr_t>(hidden) & 15u) || (reinterpret_cast<uintptr_t>(lm_head) & 15u))
        return invalid("hidden and lm_head must be 16-byte aligned");
    if (!(clip_eps >= 0.0f && clip_eps < 1.0f)) return invalid("clip_eps must be finite and in [0, 1)");
    if (!(beta >= 0.0f && beta <= 3.402823466e+38f)) return invalid("beta must be finite and non-negative");
    if (!workspace || workspace_bytes < grpo_b200_lmhead_workspace_bytes(n_rows, P) ||
        (reinterpret_cast<uintptr_t>(workspace) & 31u)) {
        set_error("workspace must be 32-byte aligned and hold grpo_b200_lmhead_workspace_bytes() bytes");
        return GRPO_B200_E_WORKSPACE;
    }
    const LmHeadPlan plan = plan_for(n_rows, P, device_sms());
    EncodeTiled encode = nullptr;
    GRPO_CUDA_TRY(encode_fn(&encode));
    CUtensorMap map_a, map_b;
    GRPO_CUDA_TRY(make_map(encode, &map_a, hidden, n_rows, C, kBM));
    GRPO_CUDA_TRY(make_map(encode, &map_b, lm_head, P, C, kBN));

    LogitsArgs a = {};
    a.logp_old = logp_old;
    a.logp_ref = logp_ref;
    a.selected = selected;
    a.advantages = advantages;
    a.weights = weights;
    a.mask = mask;
    a.n_rows = n_rows;
    a.row_offset = row_offset;
    a.tokens_per_seq = tokens_per_seq;
    a.V = V;
    a.P = P;
    a.clip_eps = clip_eps;
    a.beta = beta;
    a.rows = static_cast<RowRecord*>(workspace);
    a.selected_logp = selected_logp;
    a.result = result;
    a.status = reinterpret_cast<int*>(a.rows + n_rows);
    a.counter = reinterpret_cast<unsigned*>(a.status) + 1;
    a.partials = reinterpret_cast<double*>(reinterpret_cast<unsigned char*>(a.status) + 32);
    const size_t base = (grpo_b200_logits_workspace_bytes(n_rows) + 255) & ~static_cast<size_t>(255);

    LmHeadArgs h = {};
    h.n_rows = n_rows;
    h.V = V;
    h.P = P;
    h.C = C;
    h.n_mtiles = plan.n_mtiles;
    h.n_tiles = plan.n_tiles;
    h.n_ctas = plan.n_ctas;
    h.max_slots = plan.max_slots;
    h.selected = selected;
    h.mask = mask;
    h.partials = reinterpret_cast<float4*>(static_cast<unsigned char*>(workspace) + base);
    h.status = a.status;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    static std::mutex attr_mutex;
    static bool attr_set[64] = {false};
    {
        int dev = 0;
        GRPO_CUDA_TRY(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(attr_mutex);
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            GRPO_CUDA_TRY(cudaFuncSetAttribute(lmhead_stats_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kSmemBytes)));
            attr_set[dev] = true;
        }
    }
    GRPO_CUDA_TRY(cudaMemsetAsync(a.status, 0, 32, s));
    lmhead_stats_kernel<<<static_cast<unsigned>(plan.n_ctas), kThreads, kSmemBytes, s>>>(map_a, map_b, h);
    GRPO_CUDA_TRY(cudaGetLastError());
    lmhead_merge_kernel<<<static_cast<unsigned>((n_rows + 255) / 256), 256, 0, s>>>(h.partials, plan.n_mtiles, plan.n_tiles,
                                                                                   plan.n_ctas, a, lse_out);
    GRPO_CUDA_TRY(cudaGetLastError());
    ExchangeArgs x = {};
    GRPO_CUDA_TRY(launch_logits_reduce(a, x, s));
    return GRPO_B200_OK;
}

}  // extern "C"
