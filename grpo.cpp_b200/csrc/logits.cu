// Fused logits path (K2): log-softmax, selected-token gather, token loss and log-softmax
// backward in one pass, writing dL/dlogits over the logits.
//
// Replaces grpo_logits_fused_kernel and the three-kernel "separate" pipeline of the reference
// (src/cuda/grpo_loss_cuda.cu:181-349).  Two kernels live here.
//
// PIPELINED kernel (what GRPO_B200_LOGITS_FUSED runs whenever the layout allows):
//   * persistent: thread-block clusters of 1/2/4/8 small CTAs (four CTAs of 128 threads and 128
//     registers per SM for the common widths, so that one CTA's serial phases overlap the
//     others' work) walk the rows, every cluster taking every n-th active and every n-th masked
//     row when the caller supplies the row order, else every n-th row;
//   * a ring of shared-memory stages is filled by bulk asynchronous copies
//     (cp.async.bulk global -> shared, completion on an mbarrier) up to STAGES tiles ahead, so
//     the next rows stream in from HBM while the current row is being reduced and written back
//     -- the copy engine, not thread occupancy, hides latency.  One lane of the CTA's last warp
//     requests them at the points of a row where that warp would otherwise idle; there is no
//     producer warp, whose registers would cost every other thread a quarter of its own;
//   * each thread lifts its chunks from the ring into registers (128-bit LDS), releases the
//     stage, and keeps the row slice in registers until the gradient is stored (128-bit
//     streaming stores): one HBM read and one HBM write per logit, one exp per element;
//   * the row reduction runs registers -> warp shuffles -> one 32-byte partial per warp sent
//     with st.async into the shared memory of every CTA of the cluster, counted on that CTA's
//     mbarrier; warp 0 of every CTA combines all partials in slot order.  No global atomics.
//   Every bulk copy has a single destination CTA (its issuer).
//
// STREAMING kernel (GRPO_B200_LOGITS_SEPARATE, and any layout the pipelined kernel cannot take:
// P not a multiple of 4, unaligned base, rows beyond the largest cluster): one CTA per row,
// sweeps over global memory (max, normaliser, correction, gradient), later sweeps from L2.
//
// REDUCE kernel (second and last launch of a pass): per-row loss terms in double, fixed-order
// totals by the block that takes the last ticket, and, in sharded runs, the exchange between the
// ranks and the next pass's weights.
//
// Accuracy of the log-sum-exp.  The token loss is a cancelling sum and the reference rounds
// log p(selected) to fp32, so the normaliser has to agree with the reference's double
// arithmetic to about 1e-8 relative or rows round differently.  Both row kernels therefore
//   (1) evaluate e_i = 2^(x_i*log2e - shift) with a two-constant log2e and one FMA residual so
//       the exponent itself carries no systematic error,
//   (2) sum the e_i exactly (compensated fp32 chains, or double), combining per-warp partial
//       sums with factors good to ~5e-9 and scaling by the measured mean error of the
//       hardware ex2, and
//   (3) recompute to ~5e-9 the elements that can each carry a visible share of the normaliser
//       (every thread's two largest in the pipelined kernel; those above 1/256 of it in the
//       streaming kernel) and correct the sum.
// The pipelined kernel does (2) and (3) in float-float arithmetic (an fp32 head plus an fp32
// tail, ~48 bits): double precision gave the same digits but its dependent chains, twice per
// thread and row, cost a sixth of the kernel's bandwidth.  The streaming kernel, which is not
// bound by them, uses double.  The gradient itself only needs the fp32 e_i.
//
// Neither row kernel touches a masked row's logits or selected id; both write zeros over all P
// columns of a masked row and over columns [V, P) of an active one.
#include <cooperative_groups.h>

#include <atomic>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace grpo_b200 {

namespace {

#define kNegInf (-CUDART_INF_F)
// log2(e) split into an fp32 head and tail: kLog2eHi + kLog2eLo = log2(e) to ~1e-16
constexpr float kLog2eHi = 1.4426950216293335f;
constexpr float kLog2eLo = 1.9259629911e-8f;
constexpr double kLog2eD = 1.4426950408889634073599246810019;
constexpr double kHeavyFraction = 1.0 / 256.0;  // elements above this share of the normaliser are redone in double
// Mean relative error of ex2.approx.ftz.f32 on this architecture, measured over 4M arguments in
// [-16, -1]: -4.9e-8 (rms 5.8e-8, max 1.4e-7).  The hardware result is that much low on average,
// so sums of such terms are scaled back up; elements redone in double are exempt.
constexpr double kEx2BiasFix = 1.0 + 4.9e-8;

// e = 2^(x*log2e - shift): head product and subtraction in one FMA, tail in a second
__device__ __forceinline__ float exp_rel(float x, float shift) {
    return ex2_approx(fmaf(x, kLog2eLo, fmaf(x, kLog2eHi, -shift)));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// all-lanes double sum with a fixed butterfly (commutative pairs: same bits in every lane)
__device__ __forceinline__ double warp_sum_all(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Packed fp32x2 arithmetic (sm_100): one instruction works on two independent lanes, each with
// IEEE round-to-nearest, so the hot loops below issue half as many FMA-pipe instructions.
__device__ __forceinline__ float2 lo2(float4 v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ float2 hi2(float4 v) { return make_float2(v.z, v.w); }

// e = 2^(x*log2e - shift) on a pair
__device__ __forceinline__ float2 exp_rel2(float2 x, float2 neg_shift) {
    const float2 t = __ffma2_rn(x, make_float2(kLog2eLo, kLog2eLo), __ffma2_rn(x, make_float2(kLog2eHi, kLog2eHi), neg_shift));
    return make_float2(ex2_approx(t.x), ex2_approx(t.y));
}

// Kahan step on a pair of independent chains.  nc holds MINUS the running compensation, so that
// every operation is a packed add or a packed multiply-add by -1:
//   y = v - c;  t = s + y;  c' = (t - s) - y  <=>  nc' = (s - t) + y
__device__ __forceinline__ void kahan_add2(float2& s, float2& nc, float2 v) {
    const float2 y = __fadd2_rn(v, nc);
    const float2 t = __fadd2_rn(s, y);
    const float2 d = __ffma2_rn(t, make_float2(-1.0f, -1.0f), s);
    nc = __fadd2_rn(d, y);
    s = t;
}

__device__ __forceinline__ float max4(float4 v) { return fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }

// What the row leader hands to every thread of its CTA for the backward sweep.
struct RowBroadcast {
    float neg_g_over_z;  // -dlogp / normaliser (normaliser relative to e^M)
    float g;             // dlogp
    int selected;
};

// Per-row scalars the leader needs, fetched at the start of the row so that their latency is
// hidden behind the row's loads.
struct RowScalars {
    float lp_old, lp_ref, adv, w;
};

__device__ __forceinline__ RowScalars load_row_scalars(const LogitsArgs& a, long long row) {
    const long long seq = (a.row_offset + row) / a.tokens_per_seq;
    RowScalars r;
    r.lp_old = __ldg(a.logp_old + row);
    r.lp_ref = __ldg(a.logp_ref + row);
    r.adv = __ldg(a.advantages + seq);
    r.w = __ldg(a.weights + seq);
    return r;
}

// The row's serial section, kept short: dlogp for the backward sweep from fp32 device math
// (log, exp, expm1: a few ulp, far inside the gradient's tolerance), and the row record for the
// reduce kernel, which redoes the same step in double, off this kernel's critical path, for the
// three loss sums (a cancelling sum that needs the reference's double log-sum-exp).
// z is the normaliser relative to e^row_max.  Follows src/cpu/grpo_loss.cpp:214-215, :137-160.
// z arrives as a double or as an fp32 head + tail.
struct FF {
    float hi, lo;
};
__device__ __forceinline__ float z_as_float(double z) { return static_cast<float>(z); }
__device__ __forceinline__ float z_as_float(FF z) { return __fadd_rn(z.hi, z.lo); }
__device__ __forceinline__ double z_as_double(double z) { return z; }
__device__ __forceinline__ double z_as_double(FF z) { return static_cast<double>(z.hi) + static_cast<double>(z.lo); }
template <class Z>
__device__ __forceinline__ RowBroadcast row_leader_fast(const LogitsArgs& a, long long row, float row_max, Z z,
                                                        float x_sel, int sel, const RowScalars& sc, bool bad_input,
                                                        bool write_record) {
    const float zf = z_as_float(z);
    const float lp_new = x_sel - (row_max + logf(zf));
    const TokenTerms t = token_terms<false>(lp_new, sc.lp_old, sc.lp_ref, sc.adv, sc.w, a.clip_eps, a.beta);
    RowBroadcast b;
    b.g = t.grad;
    b.neg_g_over_z = -t.grad / zf;
    b.selected = sel;
    if (write_record) {
        RowRecord r;
        r.z = z_as_double(z);
        r.m = row_max;
        r.x_sel = x_sel;
        r.flags = bad_input ? kRowBadInput : 0.0f;
        r.pad[0] = r.pad[1] = r.pad[2] = 0.0f;
        a.rows[row] = r;
    }
    return b;
}

// ---- mbarrier / bulk-copy primitives (sm_90+ PTX) ------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: gives up after about two seconds of SM clock and reports failure, so a lost
// copy can never hang the device.  The caller then stops touching the ring ("not alive") but
// keeps meeting every block and cluster barrier until the kernel ends.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > (1LL << 32)) return false;
    }
    return true;
}
// global -> the issuing CTA's own shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// ---- float-float arithmetic: a value carried as an fp32 head plus an fp32 tail (about 48 bits).
// The per-row path of the pipelined kernel needs terms and factors good to ~1e-8 relative; double
// precision gives that, but its dependent chains sat on every thread's path twice per row and cost
// a sixth of the kernel's bandwidth.  These few fp32 instructions give the same digits.
// a + b exactly: head = fl(a + b), tail = the rounding error (symmetric in a and b, bit for bit)
__device__ __forceinline__ FF two_sum(float a, float b) {
    const float s = __fadd_rn(a, b);
    const float bb = __fsub_rn(s, a);
    return FF{s, __fadd_rn(__fsub_rn(a, __fsub_rn(s, bb)), __fsub_rn(b, bb))};
}
// a * b exactly
__device__ __forceinline__ FF two_prod(float a, float b) {
    const float p = __fmul_rn(a, b);
    return FF{p, __fmaf_rn(a, b, -p)};
}
// all-lanes float-float sum with a fixed butterfly; every step is symmetric in its two operands, so
// every lane ends with the same bits
__device__ __forceinline__ FF warp_sum_ff(FF v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oh = __shfl_xor_sync(0xffffffffu, v.hi, o);
        const float ol = __shfl_xor_sync(0xffffffffu, v.lo, o);
        const FF s = two_sum(v.hi, oh);
        v.hi = s.hi;
        v.lo = __fadd_rn(__fadd_rn(v.lo, ol), s.lo);
    }
    return v;
}

// ln 2 and (ln 2)^2 / 2 as fp32 head + tail
#define kLn2Hi 0.693147182464599609375f
#define kLn2Lo (-1.90465432314823602e-9f)
#define kHalfLn2SqHi 0.2402265071868896484375f
#define kHalfLn2SqLo (-2.27788954365593099e-10f)
// 2^(th + tl) as head + tail, |tl| tiny against |th|, th clamped to [lowest, 2] by the caller with
// lowest >= -126.  2^k * 2^r with r = t - k in [-1/2, 1/2]; 2^r = 1 + r ln2 + r^2 ln2^2/2 carried
// in float-float and the Taylor terms of degree 3 to 8 in plain fp32 (they sum to < 7e-3).
// Measured against the double-precision library over 1M arguments: 5.6e-9 relative at worst.
__device__ __forceinline__ FF exp2_ff(float th, float tl) {
    const float k = rintf(th);
    const FF r = two_sum(__fsub_rn(th, k), tl);
    const float rh = r.hi;
    float q = 1.3215486790144309e-06f;              // ln2^8 / 8!
    q = __fmaf_rn(q, rh, 1.5252733804059841e-05f);  // ln2^7 / 7!
    q = __fmaf_rn(q, rh, 1.5403530393381609e-04f);  // ln2^6 / 6!
    q = __fmaf_rn(q, rh, 1.3333558146428443e-03f);  // ln2^5 / 5!
    q = __fmaf_rn(q, rh, 9.6181291076284772e-03f);  // ln2^4 / 4!
    q = __fmaf_rn(q, rh, 5.5504108664821580e-02f);  // ln2^3 / 3!
    FF u = two_prod(rh, kLn2Hi);
    u.lo = __fmaf_rn(rh, kLn2Lo, u.lo);
    const FF v = two_prod(rh, rh);
    FF w = two_prod(v.hi, kHalfLn2SqHi);
    w.lo = __fmaf_rn(v.lo, kHalfLn2SqHi, __fmaf_rn(v.hi, kHalfLn2SqLo, w.lo));
    const float tail = __fmul_rn(__fmul_rn(v.hi, rh), q);
    const FF s1 = two_sum(1.0f, u.hi);
    const FF s2 = two_sum(s1.hi, w.hi);
    float lo = __fadd_rn(__fadd_rn(s1.lo, s2.lo), __fadd_rn(u.lo, w.lo));
    lo = __fadd_rn(lo, __fmaf_rn(r.lo, kLn2Hi, tail));
    const FF res = two_sum(s2.hi, lo);
    const float scale = __int_as_float((static_cast<int>(k) + 127) << 23);  // 2^k exactly
    return FF{__fmul_rn(res.hi, scale), __fmul_rn(res.lo, scale)};
}

// x * log2(e) - shift as head + tail: the product exactly, then an exact subtraction of the head
__device__ __forceinline__ FF scaled_minus_shift(float x, float shift) {
    const FF p = two_prod(x, kLog2eHi);
    const FF t = two_sum(p.hi, -shift);
    return FF{t.hi, __fadd_rn(t.lo, __fmaf_rn(x, kLog2eLo, p.lo))};
}

// Correction of one term given its logit: what 2^(x*log2e - shift) is to ~5e-9, minus the fp32
// term as it entered the sum (the same deterministic function as in the main sweep, so the same
// bits).  The accurate value is divided by the ex2 bias factor because the whole fp32 sum is
// multiplied by that factor later.  The two values agree to ~2e-7, so their heads subtract exactly.
// Terms below 2^-100 of the warp's largest have nothing to correct and are clamped there, which
// keeps the power of two constructible.
__device__ __forceinline__ float term_correction(float xv, float shift) {
    if (xv == kNegInf) return 0.0f;
    const FF t = scaled_minus_shift(xv, shift);
    const FF e = exp2_ff(fmaxf(t.hi, -100.0f), t.lo);
    constexpr float kInvBiasMinus1 = static_cast<float>(1.0 / kEx2BiasFix - 1.0);
    return __fadd_rn(__fsub_rn(e.hi, exp_rel(xv, shift)), __fmaf_rn(e.hi, kInvBiasMinus1, e.lo));
}

// One warp's partial of the row reduction.  Lane 0 of every consumer warp writes it into the same
// slot of EVERY CTA of the cluster (its own included) and then arrives on that CTA's exchange
// barrier, so the first thing any CTA waits for after its exponentials is the complete set.
struct __align__(16) WarpPart {
    float s_hi;   // sum of the warp's terms 2^(x*log2e - shift) as head + tail: compensated fp32 sums
    float s_lo;   // with the corrections of the dominant terms folded into the tail
    float m;      // maximum of the warp's columns (-inf when it holds none)
    float shift;  // the exponent offset the warp used
    float chk;    // finiteness probe
    float x_sel;  // the selected logit, if this warp's thread 0 found it in the CTA's slice
    int has_sel;
    int pad;
};

// Asynchronous 32-byte store of one partial into CTA `rank`'s copy of `slot`; each 16-byte half
// counts its bytes on that CTA's copy of `bar` when it lands (st.async, sm_90+).
__device__ __forceinline__ void send_part(WarpPart* slot, uint64_t* bar, unsigned rank, FF s, float m, float shift,
                                          float chk, float x_sel, int has_sel) {
    uint32_t dst, rbar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(smem_addr(slot)), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(smem_addr(bar)), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(dst),
                 "r"(__float_as_int(s.hi)), "r"(__float_as_int(s.lo)), "r"(__float_as_int(m)),
                 "r"(__float_as_int(shift)), "r"(rbar)
                 : "memory");
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(dst + 16u),
                 "r"(__float_as_int(chk)), "r"(__float_as_int(x_sel)), "r"(has_sel), "r"(0), "r"(rbar)
                 : "memory");
}

// 32 bytes of zeros with one store (256-bit stores, sm_100), marked for early eviction from L2.
// The address must be 32-byte aligned.
__device__ __forceinline__ void store_zero32(float4* p) {
    const float z = 0.0f;
    asm volatile("st.global.L2::evict_first.v8.f32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"l"(p), "f"(z) : "memory");
}

// barrier 1: all THREADS threads of the CTA (a named barrier, kept apart from __syncthreads)
__device__ __forceinline__ void consumer_sync(int threads) {
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (clock64() - start > (1LL << 32)) return false;
    }
    return true;
}

// ---------------------------------------------------------------------------------------------
// Pipelined kernel.  Requires P % 4 == 0 and 16-byte aligned bases; the dispatcher guarantees
// ceil(P/4 / CLUSTER) <= THREADS * VEC.  TJ chunks per thread per ring stage, STAGES stages.
// The block has THREADS threads; STAGES >= VEC / TJ (a whole row fits the ring).
//
// Nothing on a row's critical path is an ordinary global load: such a load queues behind the
// bulk copies this SM already has in flight and comes back thousands of cycles later.  The
// per-row scalars are staged per batch of rows, the selected logit is read back from the ring,
// and the elements that are redone accurately are the thread's own two largest chunk maxima.
// Issuing a bulk copy can itself stall for a long time when the copy queue is full, which is
// why it is done by a warp that has just handed its partial over and has nothing to do until
// the row leader is through.
// ---------------------------------------------------------------------------------------------
template <int THREADS, int VEC, int TJ, int STAGES, int CLUSTER, int MINB, bool CHECK>
__global__ void __launch_bounds__(THREADS, MINB) logits_pipelined_kernel(const LogitsArgs a) {
    constexpr int WARPS = THREADS / 32;
    constexpr int TILE_CHUNKS = TJ * THREADS;
    constexpr int TILES = VEC / TJ;
    constexpr int BATCH = 128;  // rows whose scalars are staged at once
    static_assert(VEC % TJ == 0, "tiles must cover the per-thread chunks exactly");
    static_assert(STAGES >= VEC / TJ, "the ring holds at least one whole row slice");
    static_assert(WARPS <= 32, "warp indices fit one lane each");

    extern __shared__ __align__(128) unsigned char ring_raw[];
    float4* ring = reinterpret_cast<float4*>(ring_raw);
    __shared__ uint64_t full_bar[STAGES];
    __shared__ uint64_t empty_bar[STAGES];
    __shared__ uint64_t xbar[2];                    // [row parity]: completes when all CLUSTER * WARPS partials are in
    __shared__ WarpPart parts[2][CLUSTER * WARPS];  // [row parity][source rank * WARPS + source warp]
    __shared__ float warp_f[WARPS];  // 2^(shift_w - M*log2e): the warp's terms relative to the row maximum
    __shared__ RowBroadcast bc;
    __shared__ int meta_sel[BATCH];
    __shared__ float meta_old[BATCH];
    __shared__ float meta_ref[BATCH];
    __shared__ float meta_adv[BATCH];
    __shared__ float meta_w[BATCH];
    __shared__ unsigned char meta_mask[BATCH];
    __shared__ int meta_row[BATCH];
    __shared__ unsigned q_cons_final;
    __shared__ int abort_sh;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    // The reduce kernel that follows in the stream may be made resident as this grid's CTAs retire
    // and run its prologue; it still waits for this whole grid before it reads anything written here.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // The pass's control words start from zero without a separate clearing launch: block 0 is
    // resident from the first instant (the grid never exceeds what fits at once), CTAs report into
    // the status word only when they retire, and the reduce kernel that reads both runs after this kernel.
    if (blockIdx.x == 0 && tid == 0) {
        *a.status = 0;
        *a.counter = 0u;
    }
    // the row order's two counts, requested now so that their latency overlaps the start-up barriers below
    const int* order = a.row_order;
    int order_active = 0, order_masked = 0;
    if (order) {
        order_active = __ldg(order);
        order_masked = __ldg(order + 1);
    }
    unsigned crank = 0;
    if (CLUSTER > 1) crank = cg::this_cluster().block_rank();
    const int cluster_id = blockIdx.x / CLUSTER;
    const int n_clusters = gridDim.x / CLUSTER;
    const int n_rows = static_cast<int>(a.n_rows);  // the C ABI caps rows at INT_MAX

    const int V = a.V;
    const int P4 = a.P >> 2;
    const int per_cta = (P4 + CLUSTER - 1) / CLUSTER;
    const int c0 = static_cast<int>(crank) * per_cta;        // first chunk of this CTA's slice
    const int n_store = max(min(c0 + per_cta, P4) - c0, 0);  // chunks of the slice (stores)
    const int n_load = max(min(c0 + n_store, (V + 3) >> 2) - c0, 0);  // chunks that hold vocabulary (loads)
    const int n_tiles = (n_load + TILE_CHUNKS - 1) / TILE_CHUNKS;
    // masked rows are zero-filled with 256-bit stores when every row's slice starts on a 32-byte boundary
    const bool wide_fill = (a.P & 7) == 0 && (c0 & 1) == 0 && (reinterpret_cast<uintptr_t>(a.dlogits) & 31u) == 0;
    // The single chunk that straddles column V (when V % 4 != 0) belongs to one thread of one CTA:
    // special_j is its register index there, -1 everywhere else.
    const int v_rem = V & 3;
    int special_j = -1;
    if (v_rem != 0) {
        const int cs = (V >> 2) - c0;
        if (cs >= 0 && cs < n_store && cs % THREADS == tid) special_j = cs / THREADS;
    }

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], WARPS);
        }
        // one CTA: WARPS plain arrivals; a cluster: one arrival that announces the bytes, the bytes count themselves
        for (int i = 0; i < 2; i++) mbar_init(&xbar[i], CLUSTER == 1 ? WARPS : 1);
        q_cons_final = 0;
        abort_sh = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (CLUSTER > 1) cg::this_cluster().sync();  // peers' barriers exist before anyone arrives on them remotely

    // Rows of this cluster.  Without a row order: cluster_id + k * n_clusters, k = 0 .. n_mine-1,
    // whatever their masks.  With one (row_order = {n_active, n_masked, active rows..., masked
    // rows...}): every n_clusters-th ACTIVE row and every n_clusters-th MASKED row, so that all
    // clusters carry the same load to within a row, interleaved evenly (slot k is an active row
    // when floor((k+1) * mine_active / n_mine) steps up) so that zero fills keep overlapping with
    // the active rows' phases.
    // A row order whose two counts do not add up to the row count belongs to another batch: it is
    // ignored (every CTA reads the same two words, so the decision is uniform) and the pass reports it.
    if (order) {
        const int na = order_active, nm = order_masked;
        if (na < 0 || nm < 0 || static_cast<long long>(na) + nm != a.n_rows) {
            order = nullptr;
            if (blockIdx.x == 0 && tid == 0) atomicOr(&abort_sh, kStatusRowOrderMismatch);
        }
    }
    const int total_active = order ? order_active : 0;
    const int total_masked = order ? order_masked : 0;
    const int* active_rows = order ? order + 2 : nullptr;
    const int* masked_rows = order ? order + 2 + total_active : nullptr;
    const int mine_active = order && cluster_id < total_active ? (total_active - cluster_id + n_clusters - 1) / n_clusters : 0;
    const int mine_masked = order && cluster_id < total_masked ? (total_masked - cluster_id + n_clusters - 1) / n_clusters : 0;
    const int n_mine = order ? mine_active + mine_masked
                             : (cluster_id < n_rows ? (n_rows - cluster_id + n_clusters - 1) / n_clusters : 0);

    unsigned q = 0;     // tiles consumed
    bool alive = true;  // false after a wait timed out: skip the ring, keep meeting barriers
    // Lane 0 of the last warp requests the tiles, at the two points where that warp has nothing
    // else to do: when a batch of rows has been staged (it fills the ring) and right after its
    // hand-over of a row (it refills the stages that row gave back, while warp 0 combines and runs
    // the leader).  It walks the staged rows of the current batch only, so the ring runs dry at a
    // batch's end: one memory latency per BATCH rows.
    const bool is_issuer = warp == WARPS - 1 && lane == 0;
    int p_slot = 0, p_tile = 0;  // next row of the batch and next tile of it to request
    unsigned q_prod = 0;         // tiles requested
    unsigned row_parity = 0;
    unsigned xuses[2] = {0u, 0u};

    // request up to `budget` more tiles of the current batch's active rows, in the order the consumers take them
    auto issue_tiles = [&](int budget, int batch_rows) {
        while (budget > 0) {
            while (p_slot < batch_rows && meta_mask[p_slot] != 1) p_slot++;
            if (p_slot >= batch_rows) break;
            const unsigned slot = q_prod % STAGES;
            const unsigned parity = (q_prod / STAGES) & 1u;
            if (!mbar_wait(&empty_bar[slot], parity ^ 1u)) {
                atomicOr(&abort_sh, kStatusPipelineTimeout);
                p_slot = batch_rows;  // request nothing more: the consumers' waits run out and report
                break;
            }
            const float* row_src = a.logits + static_cast<size_t>(meta_row[p_slot]) * static_cast<size_t>(a.P) +
                                   4 * static_cast<size_t>(c0);
            const int first = p_tile * TILE_CHUNKS;
            const uint32_t bytes = static_cast<uint32_t>(min(TILE_CHUNKS, n_load - first)) * 16u;
            mbar_arrive_expect_tx(&full_bar[slot], bytes);
            bulk_load(ring + static_cast<size_t>(slot) * TILE_CHUNKS, row_src + 4 * static_cast<size_t>(first), bytes,
                      &full_bar[slot]);
            q_prod++;
            budget--;
            if (++p_tile == n_tiles) {
                p_tile = 0;
                p_slot++;
            }
        }
    };

    for (int batch_first = 0; batch_first < n_mine; batch_first += BATCH) {
        const int batch_rows = min(BATCH, n_mine - batch_first);
        consumer_sync(THREADS);  // every consumer is done with the previous batch's scalars
        for (int i = tid; i < batch_rows; i += THREADS) {
            const long long k = batch_first + i;
            size_t r = static_cast<size_t>(cluster_id) + static_cast<size_t>(k) * n_clusters;
            int mk;
            if (order) {
                const long long before = k * mine_active / n_mine;  // active rows among this cluster's first k
                mk = (k + 1) * mine_active / n_mine > before;
                const size_t nth = mk ? static_cast<size_t>(before) : static_cast<size_t>(k - before);
                const int listed = (mk ? active_rows : masked_rows)[static_cast<size_t>(cluster_id) + nth * n_clusters];
                // the list must name rows of this batch and agree with the mask the reduce kernel reads;
                // a row it misplaces is skipped (nothing loaded, nothing stored) and the pass reports it
                if (listed < 0 || listed >= n_rows) {
                    mk = 2;
                    r = 0;
                    atomicOr(&abort_sh, kStatusRowOrderMismatch);
                } else {
                    r = static_cast<size_t>(listed);  // checked against the mask below, off the path to the first request
                }
            } else {
                mk = a.mask[r] != 0;
            }
            meta_row[i] = static_cast<int>(r);
            meta_mask[i] = static_cast<unsigned char>(mk);
        }
        consumer_sync(THREADS);
        // Every tile requested so far has been consumed: the ring is empty, and the new batch's rows
        // are known.  The first tiles are requested now, so that they travel while the rows' scalars
        // are being fetched.
        p_slot = 0;
        p_tile = 0;
        if (is_issuer && n_tiles > 0) issue_tiles(STAGES, batch_rows);
        for (int i = tid; i < batch_rows; i += THREADS) {
            if (order && meta_mask[i] != 2 && (a.mask[meta_row[i]] != 0) != (meta_mask[i] != 0))
                atomicOr(&abort_sh, kStatusRowOrderMismatch);
            if (meta_mask[i] == 1) {
                const size_t r = static_cast<size_t>(meta_row[i]);
                const long long seq = (a.row_offset + static_cast<long long>(r)) / a.tokens_per_seq;
                meta_sel[i] = a.selected[r];
                meta_old[i] = a.logp_old[r];
                meta_ref[i] = a.logp_ref[r];
                meta_adv[i] = a.advantages[seq];
                meta_w[i] = a.weights[seq];
            }
        }
        consumer_sync(THREADS);

        // ---- consumer warps
        for (int k_row = 0; k_row < batch_rows; k_row++) {
            const size_t row = static_cast<size_t>(meta_row[k_row]);
            float4* out = reinterpret_cast<float4*>(a.dlogits + row * static_cast<size_t>(a.P)) + c0;

            if (meta_mask[k_row] == 2) continue;  // a row index outside the batch: neither loaded nor stored
            if (meta_mask[k_row] == 0) {  // uniform over the cluster: no barrier is reached
                const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (wide_fill) {
                    const int pairs = n_store >> 1;
#pragma unroll
                    for (int j = 0; j < VEC / 2; j++) {
                        const int local = j * THREADS + tid;
                        if (local < pairs) store_zero32(out + 2 * local);
                    }
                    if ((n_store & 1) && tid == 0) store_stream(out + n_store - 1, zero);
                } else {
#pragma unroll
                    for (int j = 0; j < VEC; j++) {
                        const int local = j * THREADS + tid;
                        if (local < n_store) store_stream(out + local, zero);
                    }
                }
                continue;
            }

            // ---- ring -> registers, one stage at a time
            const int slot0 = static_cast<int>(q % STAGES);
            float4 x[VEC];
#pragma unroll
            for (int k = 0; k < TILES; k++) {
                if (k < n_tiles) {
                    const unsigned slot = q % STAGES;
                    const unsigned parity = (q / STAGES) & 1u;
                    if (alive) alive = mbar_wait(&full_bar[slot], parity);
                    const float4* stage = ring + static_cast<size_t>(slot) * TILE_CHUNKS;
#pragma unroll
                    for (int jj = 0; jj < TJ; jj++) {
                        const int local = k * TILE_CHUNKS + jj * THREADS + tid;
                        if (alive && local < n_load)
                            x[k * TJ + jj] = stage[jj * THREADS + tid];
                        else
                            x[k * TJ + jj] = make_float4(kNegInf, kNegInf, kNegInf, kNegInf);
                    }
                    q++;
                } else {
#pragma unroll
                    for (int jj = 0; jj < TJ; jj++) x[k * TJ + jj] = make_float4(kNegInf, kNegInf, kNegInf, kNegInf);
                }
            }

            // ---- the selected logit, read back from the stage that holds its chunk
            int sel = 0;
            float x_sel = 0.0f;
            int has_sel = 0;
            bool bad_sel = false;
            if (tid == 0) {
                sel = meta_sel[k_row];
                if (sel < 0 || sel >= V) {  // the host layer rejects this earlier; never read out of the row
                    bad_sel = true;
                    sel = 0;
                }
                const int sc = (sel >> 2) - c0;
                if (alive && sc >= 0 && sc < n_load) {
                    int slot = slot0 + sc / TILE_CHUNKS;
                    if (slot >= STAGES) slot -= STAGES;
                    const float* stage = reinterpret_cast<const float*>(ring + static_cast<size_t>(slot) * TILE_CHUNKS);
                    x_sel = stage[4 * (sc % TILE_CHUNKS) + (sel & 3)];
                    has_sel = 1;
                }
            }

            // ---- the row's stages are free again; the issuing lane refills them after the hand-over below
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < TILES; k++) {
                    if (k < n_tiles) {
                        int slot = slot0 + k;
                        if (slot >= STAGES) slot -= STAGES;
                        mbar_arrive(&empty_bar[slot]);
                    }
                }
            }

            // ---- padding columns of the chunk that straddles V, finiteness probe, and the thread's
            //      two largest chunk maxima (its candidates for the accurate correction)
            if (special_j >= 0) {  // the one thread that owns the chunk holding column V
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    if (j == special_j) {
                        if (v_rem < 2) x[j].y = kNegInf;
                        if (v_rem < 3) x[j].z = kNegInf;
                        x[j].w = kNegInf;
                    }
                }
            }
            float chk = 0.0f;
            float m = kNegInf, m2 = kNegInf;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                // uniform test, made only inside the last tile so that the chunks before it schedule as one block:
                // does chunk index j hold columns for any thread of this CTA?
                if (j < VEC - TJ || j * THREADS < n_load) {
                    if (CHECK) {
                        // x * 0 is NaN for an infinite or NaN logit and 0 otherwise; -inf marks "no column here"
                        if (x[j].x != kNegInf) chk = fmaf(x[j].x, 0.0f, chk);
                        if (x[j].y != kNegInf) chk = fmaf(x[j].y, 0.0f, chk);
                        if (x[j].z != kNegInf) chk = fmaf(x[j].z, 0.0f, chk);
                        if (x[j].w != kNegInf) chk = fmaf(x[j].w, 0.0f, chk);
                    }
                    const float cm = max4(x[j]);
                    m2 = fmaxf(m2, fminf(m, cm));
                    m = fmaxf(m, cm);
                }
            }

            // ---- one exp per element relative to the warp's maximum; compensated fp32 sums (four
            //      independent Kahan chains, two per packed instruction) keep the thread's total
            //      exact to about 48 bits
            const float m_warp = warp_max(m);
            const float shift = (m_warp == kNegInf ? 0.0f : m_warp) * kLog2eHi;
            const float2 neg_shift2 = make_float2(-shift, -shift);
            float2 sa = make_float2(0.0f, 0.0f), nca = sa, sb = sa, ncb = sa;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                if (j < VEC - TJ || j * THREADS < n_load) {
                    const float2 ea = exp_rel2(lo2(x[j]), neg_shift2);
                    const float2 eb = exp_rel2(hi2(x[j]), neg_shift2);
                    x[j] = make_float4(ea.x, ea.y, eb.x, eb.y);
                    kahan_add2(sa, nca, ea);
                    kahan_add2(sb, ncb, eb);
                }
            }
            // the thread's total as head + tail: the four sums add exactly (two_sum), their
            // compensations and rounding errors collect in the tail
            const FF t01 = two_sum(sa.x, sa.y), t23 = two_sum(sb.x, sb.y);
            const FF t4 = two_sum(t01.hi, t23.hi);
            float s_tail = __fadd_rn(__fadd_rn(__fadd_rn(nca.x, nca.y), __fadd_rn(ncb.x, ncb.y)),
                                     __fadd_rn(__fadd_rn(t01.lo, t23.lo), t4.lo));
            // Every thread redoes its two largest chunk maxima to ~5e-9: a row's few dominant terms
            // are among them, and those are the terms whose fp32 error (~1e-7 each) the
            // log-sum-exp cannot absorb.  Everything else is light enough to average out.
            s_tail = __fadd_rn(s_tail, __fadd_rn(term_correction(m, shift), term_correction(m2, shift)));
            const FF s_warp = warp_sum_ff(FF{t4.hi, s_tail});
            if (CHECK) chk = warp_sum_f(chk);

            // ---- every warp hands its partial to every CTA of the cluster: lane p sends it to CTA p
            //      with asynchronous stores that count their bytes on CTA p's exchange barrier, so the
            //      sender waits for nothing
            if (CLUSTER == 1) {
                if (lane == 0) {
                    WarpPart mine;
                    mine.s_hi = s_warp.hi;
                    mine.s_lo = s_warp.lo;
                    mine.m = m_warp;
                    mine.shift = shift;
                    mine.chk = chk;
                    mine.x_sel = x_sel;  // zero except in thread 0
                    mine.has_sel = has_sel;
                    mine.pad = 0;
                    parts[row_parity][warp] = mine;
                    mbar_arrive(&xbar[row_parity]);
                }
            } else {
                const float xs0 = __shfl_sync(0xffffffffu, x_sel, 0);  // zero except in warp 0
                const int hs0 = __shfl_sync(0xffffffffu, has_sel, 0);
                if (tid == 0) mbar_arrive_expect_tx(&xbar[row_parity], CLUSTER * WARPS * sizeof(WarpPart));
                if (lane < CLUSTER)
                    send_part(&parts[row_parity][crank * WARPS + warp], &xbar[row_parity], static_cast<unsigned>(lane),
                              s_warp, m_warp, shift, chk, xs0, hs0);
            }

            if (is_issuer && n_tiles > 0) issue_tiles(n_tiles, batch_rows);  // the stages this row gave back

            // ---- warp 0 of every CTA combines all partials of the row: same slots, same order,
            //      same bits in every CTA.  Factors and sums in float-float, fixed shuffle trees.
            if (warp == 0) {
                constexpr int PARTS = CLUSTER * WARPS;
                constexpr int PER_LANE = (PARTS + 31) / 32;
                if (alive)
                    alive = CLUSTER > 1 ? mbar_wait_cluster(&xbar[row_parity], xuses[row_parity] & 1u)
                                        : mbar_wait(&xbar[row_parity], xuses[row_parity] & 1u);
                xuses[row_parity]++;
                const WarpPart* in = parts[row_parity];
                float m_lane = kNegInf;
#pragma unroll
                for (int i = 0; i < PER_LANE; i++) {
                    const int idx = lane + 32 * i;
                    if (idx < PARTS) m_lane = fmaxf(m_lane, in[idx].m);
                }
                const float m_row = warp_max(m_lane);
                // m_row * log2(e) as head + tail
                const FF row_shift_p = two_prod(m_row, kLog2eHi);
                const float row_shift_lo = __fmaf_rn(m_row, kLog2eLo, row_shift_p.lo);
                FF s = FF{0.0f, 0.0f};
                float c = 0.0f, xs = 0.0f;
#pragma unroll
                for (int i = 0; i < PER_LANE; i++) {
                    const int idx = lane + 32 * i;
                    if (idx < PARTS) {
                        const WarpPart part = in[idx];
                        // the warp's terms are 2^(x*log2e - shift); relative to e^m_row they scale by
                        // f = 2^(shift - m_row*log2e) * (ex2 bias factor).  Warps more than 2^-120
                        // below the row maximum are clamped there: they cannot reach the sum.
                        FF f = FF{0.0f, 0.0f};
                        if (part.m != kNegInf) {
                            const FF d = two_sum(part.shift, -row_shift_p.hi);
                            f = exp2_ff(fmaxf(d.hi, -120.0f), __fsub_rn(d.lo, row_shift_lo));
                            f.lo = __fmaf_rn(f.hi, static_cast<float>(kEx2BiasFix - 1.0), f.lo);
                        }
                        // s += part.s * f in float-float
                        const FF ph = two_prod(part.s_hi, f.hi);
                        const float pl = __fmaf_rn(part.s_hi, f.lo, __fmaf_rn(part.s_lo, f.hi, ph.lo));
                        const FF acc = two_sum(s.hi, ph.hi);
                        s.hi = acc.hi;
                        s.lo = __fadd_rn(__fadd_rn(s.lo, pl), acc.lo);
                        if (CHECK) c += part.chk;
                        if (part.has_sel) xs += part.x_sel;  // exactly one warp of the cluster holds it
                        if (idx / WARPS == static_cast<int>(crank)) warp_f[idx % WARPS] = __fadd_rn(f.hi, f.lo);
                    }
                }
                const FF z_row = warp_sum_ff(s);
                if (CHECK) c = warp_sum_f(c);
                x_sel = warp_sum_f(xs);
                // ---- row leader: dlogp for the backward sweep and the row's record.  Every CTA of
                //      the cluster repeats it on the same bits; rank 0 writes the record.
                if (lane == 0)
                    bc = row_leader_fast(a, static_cast<long long>(row), m_row, z_row, x_sel, sel,
                                         RowScalars{meta_old[k_row], meta_ref[k_row], meta_adv[k_row], meta_w[k_row]},
                                         bad_sel || (CHECK && c != 0.0f) || !alive, crank == 0);
            }
            consumer_sync(THREADS);
            // ---- backward sweep from registers: g * (onehot - p) = e_i * coef + [i == sel] * g
            const RowBroadcast b = bc;
            const float coef = warp_f[warp] * b.neg_g_over_z;
            if (special_j >= 0) {  // padding columns inside the chunk that straddles V come back as +0
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    if (j == special_j) {
                        if (v_rem < 2) x[j].y = 0.0f;
                        if (v_rem < 3) x[j].z = 0.0f;
                        x[j].w = 0.0f;
                    }
                }
            }
            float e_sel = 0.0f;  // the selected column's term, if this thread holds it
            const int sel_local = (b.selected >> 2) - c0;
            const bool owns_sel = sel_local >= 0 && sel_local < n_load && sel_local % THREADS == tid;
            if (owns_sel) {
                const int j_sel = sel_local / THREADS, q_sel = b.selected & 3;
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    if (j == j_sel) e_sel = q_sel == 0 ? x[j].x : q_sel == 1 ? x[j].y : q_sel == 2 ? x[j].z : x[j].w;
                }
            }
            const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float2 coef2 = make_float2(coef, coef);
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                const int local = j * THREADS + tid;
                if (local < n_store) {
                    float4 o = zero;  // columns [V, P) of the slice
                    if (local < n_load) {
                        const float2 oa = __fmul2_rn(lo2(x[j]), coef2), ob = __fmul2_rn(hi2(x[j]), coef2);
                        o = make_float4(oa.x, oa.y, ob.x, ob.y);
                    }
                    store_stream(out + local, o);
                }
            }
            // same thread, same address, program order: this store lands after the vector store above
            if (owns_sel) a.dlogits[row * static_cast<size_t>(a.P) + b.selected] = fmaf(e_sel, coef, b.g);
            row_parity ^= 1u;
        }  // rows of the batch
    }      // batches

    // ---- shutdown: nothing may still be landing in this CTA's shared memory when it retires
    if (tid == 0) q_cons_final = q;
    if (!alive) atomicOr(&abort_sh, kStatusPipelineTimeout);
    __syncthreads();
    if (is_issuer) {
        unsigned qc = q_cons_final;
        while (qc < q_prod) {  // requested but never consumed (only after a timeout)
            mbar_wait(&full_bar[qc % STAGES], (qc / STAGES) & 1u);
            qc++;
        }
        // the pass's status word was cleared by block 0's first instruction, long before any CTA gets here
        if (abort_sh != 0) atomicOr(a.status, abort_sh);
    }
    if (CLUSTER > 1) cg::this_cluster().sync();  // no CTA retires while a peer may still push into its inbox
}

// ---------------------------------------------------------------------------------------------
// Streaming kernel: one CTA per row, any V / P / alignment.
// ---------------------------------------------------------------------------------------------
constexpr int kStreamThreads = 512;

template <bool CHECK>
__global__ void __launch_bounds__(kStreamThreads) logits_streaming_kernel(const LogitsArgs a) {
    constexpr int WARPS = kStreamThreads / 32;
    __shared__ float red[WARPS];
    __shared__ float red_chk[WARPS];
    __shared__ double red_d[WARPS];
    __shared__ double z_sh;
    __shared__ RowBroadcast bc;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long row = blockIdx.x;
    const float* in = a.logits + row * static_cast<long long>(a.P);
    float* out = a.dlogits + row * static_cast<long long>(a.P);
    const int V = a.V, P = a.P;
    // the pass's control words start from zero (this kernel never sets the status word; the reduce
    // kernel, which runs after it, reads both)
    if (blockIdx.x == 0 && tid == 0) {
        *a.status = 0;
        *a.counter = 0u;
    }

    if (a.mask[row] == 0) {
        for (int v = tid; v < P; v += kStreamThreads) out[v] = 0.0f;
        return;
    }

    // sweep 1: maximum (and the finiteness probe)
    float m = kNegInf, chk = 0.0f;
    for (int v = tid; v < V; v += kStreamThreads) {
        const float x = in[v];
        m = fmaxf(m, x);
        if (CHECK) chk = fmaf(x, 0.0f, chk);
    }
    m = warp_max(m);
    if (CHECK) chk = warp_sum_f(chk);
    if (lane == 0) {
        red[warp] = m;
        if (CHECK) red_chk[warp] = chk;
    }
    __syncthreads();
    m = red[0];
    chk = CHECK ? red_chk[0] : 0.0f;
#pragma unroll
    for (int k = 1; k < WARPS; k++) {
        m = fmaxf(m, red[k]);
        if (CHECK) chk += red_chk[k];
    }

    // sweep 2: normaliser in double; terms are 2^(x*log2e - shift), rescaled to e^m once at the end
    const float shift = m * kLog2eHi;
    const double f_d = exp2(static_cast<double>(shift) - static_cast<double>(m) * kLog2eD) * kEx2BiasFix;
    double s = 0.0;
    for (int v = tid; v < V; v += kStreamThreads) s += static_cast<double>(exp_rel(in[v], shift));
    s = warp_sum_all(s);
    if (lane == 0) red_d[warp] = s;
    __syncthreads();
    if (tid == 0) {
        double z = 0.0;
#pragma unroll
        for (int k = 0; k < WARPS; k++) z += red_d[k];
        z_sh = z * f_d;
    }
    __syncthreads();
    double z = z_sh;

    // sweep 3 (rows with heavy elements only): redo those elements in double
    if (z < 1.0 / kHeavyFraction) {
        const float cut = static_cast<float>(z * kHeavyFraction * 0.999 / f_d);
        double delta = 0.0;
        for (int v = tid; v < V; v += kStreamThreads) {
            const float x = in[v];
            const float e = exp_rel(x, shift);
            if (e >= cut) delta += exp(static_cast<double>(x) - static_cast<double>(m)) - static_cast<double>(e) * f_d;
        }
        delta = warp_sum_all(delta);
        __syncthreads();  // red_d is reused
        if (lane == 0) red_d[warp] = delta;
        __syncthreads();
        if (tid == 0) {
            double d = 0.0;
#pragma unroll
            for (int k = 0; k < WARPS; k++) d += red_d[k];
            z_sh = z + d;
        }
        __syncthreads();
        z = z_sh;
    }

    if (tid == 0) {
        int sel = a.selected[row];
        bool bad = CHECK && chk != 0.0f;
        if (sel < 0 || sel >= V) {
            bad = true;
            sel = 0;
        }
        bc = row_leader_fast(a, row, m, z, in[sel], sel, load_row_scalars(a, row), bad, true);
    }
    __syncthreads();

    // last sweep: gradient; each element is read and then overwritten by the same thread
    const RowBroadcast b = bc;
    const float coef = b.neg_g_over_z * static_cast<float>(f_d);
    for (int v = tid; v < V; v += kStreamThreads) {
        const float e = exp_rel(in[v], shift);
        out[v] = e * coef + (v == b.selected ? b.g : 0.0f);
    }
    for (int v = V + tid; v < P; v += kStreamThreads) out[v] = 0.0f;
}

// Reduce kernel, the second and last launch of a pass.
//
// 1. One thread per row redoes the row's scalar step in double -- log-sum-exp, log p(selected)
//    rounded to fp32 exactly as the reference rounds it, the two exponentials -- and each block of
//    1,024 rows leaves its five sums (fixed tree) in its own slot of the workspace (a launch of a
//    single block keeps them in registers and skips step 2's round trip).  Sharded runs:
//    the same threads count the next pass's valid tokens per response (integer atomics: exact,
//    so order does not matter) into the rank's exchange region.
// 2. The block that finishes last (a ticket counter; no floating-point atomics anywhere) adds the
//    slots in index order, so the totals depend on the row count only, never on scheduling.
// 3. Sharded runs: the same block then carries out the pass's only exchange itself.  It writes
//    the record, followed by this rank's counts, into its slot of every rank's exchange region
//    over NVLink -- 8-byte words that carry the pass number next to 32 bits of data, so no fence
//    and no separate flag -- polls (bounded) its own region until every rank's words show this
//    pass's number, adds the slots in rank order -- the same bits on every rank -- and derives
//    the next pass's weights from the global counts.  A non-zero
//    status word (a pipeline wait timed out) turns bad_inputs into -1, an exchange that timed
//    out into -2.
constexpr int kReduceThreads = 1024;

__device__ __forceinline__ unsigned long long* exchange_slot(unsigned char* region, long long stride, int buf, int src) {
    return reinterpret_cast<unsigned long long*>(region + kExchangeHeaderBytes) + (buf * kExchangeMaxWorld + src) * stride * 2;
}

__global__ void __launch_bounds__(kReduceThreads) logits_reduce_kernel(const LogitsArgs a, const ExchangeArgs x) {
    __shared__ double scratch[5 * kReduceThreads / 32];
    __shared__ double record[5];
    __shared__ int hist[kReduceThreads + 1];
    __shared__ int is_last, timed_out;
    __shared__ unsigned long long pass_sh;
    const int tid = threadIdx.x;
    const long long first_row = static_cast<long long>(blockIdx.x) * kReduceThreads;
    const long long row = first_row + tid;

    // ---- the next pass's valid tokens per response among this block's rows
    if (x.world > 0) {
        const long long first_seq = (a.row_offset + first_row) / a.tokens_per_seq;
        hist[tid] = 0;
        if (tid == 0) hist[kReduceThreads] = 0;
        __syncthreads();
        if (row < a.n_rows && x.next_mask[row] != 0)
            atomicAdd(&hist[static_cast<int>((a.row_offset + row) / a.tokens_per_seq - first_seq)], 1);
        __syncthreads();
        int32_t* counts = reinterpret_cast<int32_t*>(x.peers[x.rank] + exchange_counts_offset(x.n_seq));
        for (int i = tid; i <= kReduceThreads; i += kReduceThreads)
            if (hist[i] != 0) atomicAdd(counts + first_seq + i, hist[i]);
    }

    // Everything above and the loads just below depend on nothing the row kernel writes: they may run
    // while its last CTAs are still working (programmatic dependent launch).  From here on its
    // records, status word and cleared ticket counter are needed.
    // (a null mask: a lengths-only exchange, launched on its own with no rows to reduce)
    const bool row_active = a.mask != nullptr && row < a.n_rows && a.mask[row] != 0;
    RowScalars sc = {0.0f, 0.0f, 0.0f, 0.0f};
    if (row_active) sc = load_row_scalars(a, row);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    double v[5] = {0.0, 0.0, 0.0, 0.0, 0.0};
    if (row < a.n_rows) {
        float lp_new = 0.0f;
        if (row_active) {
            const RowRecord r = a.rows[row];
            const double lse = static_cast<double>(r.m) + log(r.z);
            lp_new = static_cast<float>(static_cast<double>(r.x_sel) - lse);
            const TokenTerms t = token_terms<true>(lp_new, sc.lp_old, sc.lp_ref, sc.adv, sc.w, a.clip_eps, a.beta);
            v[0] = static_cast<double>(t.loss);
            v[1] = static_cast<double>(t.pg);
            v[2] = static_cast<double>(t.kl);
            if (!finite_f(t.grad) || !finite_f(t.grad / static_cast<float>(r.z))) v[3] = 1.0;
            if (r.flags != 0.0f) v[4] = 1.0;
        }
        if (a.selected_logp) a.selected_logp[row] = lp_new;
    }
    block_sum<kReduceThreads, 5>(v, scratch);
    double t[5] = {0.0, 0.0, 0.0, 0.0, 0.0};
    if (gridDim.x == 1) {
        // a launch of one block (up to 1,024 rows) has its totals already: no slot, no ticket, no second
        // round trip through memory -- the same bits as the general path gives for one slot
        if (tid == 0) timed_out = 0;
#pragma unroll
        for (int k = 0; k < 5; k++) t[k] = v[k] + 0.0;  // as the general path's additions of zero leave it (-0 becomes +0)
        __syncthreads();
    } else {
        if (tid == 0) {
#pragma unroll
            for (int k = 0; k < 5; k++) a.partials[static_cast<size_t>(blockIdx.x) * 5 + k] = v[k];
            __threadfence();  // the slot and this block's counts are visible before the ticket is taken
            is_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
            timed_out = 0;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        for (unsigned b = tid; b < gridDim.x; b += kReduceThreads) {
#pragma unroll
            for (int k = 0; k < 5; k++) t[k] += __ldcg(a.partials + static_cast<size_t>(b) * 5 + k);
        }
        block_sum<kReduceThreads, 5>(t, scratch);
    }
    if (tid == 0) {
        const int status = *a.status;
        if (status & kStatusRowOrderMismatch) t[4] = kBadInputsRowOrder;
        if (status & kStatusPipelineTimeout) t[4] = kBadInputsPipelineTimeout;
        if (x.world <= 0) {
            a.result->loss = t[0];
            a.result->pg_loss = t[1];
            a.result->kl = t[2];
            a.result->bad_grads = t[3];
            a.result->bad_inputs = t[4];
        }
#pragma unroll
        for (int k = 0; k < 5; k++) record[k] = t[k];
        if (x.world > 0) {
            // this region's pass number, counted on the device so that a recorded launch can be replayed;
            // every rank makes the same calls, so the ranks' counters agree
            unsigned long long* counter = reinterpret_cast<unsigned long long*>(x.peers[x.rank] + kExchangePassOffset);
            pass_sh = *counter + 1ULL;
            *counter = pass_sh;
        }
    }
    if (x.world <= 0) return;
    __syncthreads();

    // ---- the exchange: push (clearing the counts for the next pass), poll, add.  Every double
    //      travels as two 8-byte words, each carrying 32 bits of it next to the pass number: an
    //      8-byte store arrives whole, so a word that shows this pass's number is this pass's
    //      data and no fence or separate flag is needed.
    const unsigned long long seq = pass_sh;
    const unsigned long long tag = (seq & 0xffffffffULL) << 32;  // never zero-matching: the region starts zeroed, seq >= 1
    const int buf = static_cast<int>(seq & 1ULL);
    const long long n = 5 + x.n_seq;
    const long long stride = exchange_stride(x.n_seq);
    int32_t* counts = reinterpret_cast<int32_t*>(x.peers[x.rank] + exchange_counts_offset(x.n_seq));
    for (long long i = tid; i < n; i += kReduceThreads) {
        double mine = 0.0;
        if (i < 5) {
            mine = record[i];
        } else {
            mine = static_cast<double>(__ldcg(counts + (i - 5)));
            counts[i - 5] = 0;
        }
        const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(mine));
        const unsigned long long w0 = (bits & 0xffffffffULL) | tag, w1 = (bits >> 32) | tag;
        for (int p = 0; p < x.world; p++) {
            unsigned long long* dst = exchange_slot(x.peers[p], stride, buf, x.rank) + 2 * i;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(w0) : "memory");
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 1), "l"(w1) : "memory");
        }
    }
    double* out = reinterpret_cast<double*>(a.result);
    double* global_lengths = reinterpret_cast<double*>(x.peers[x.rank] + exchange_lengths_offset(x.n_seq));
    const long long start = clock64();
    for (long long i = tid; i < n; i += kReduceThreads) {
        double s = 0.0;
        double worst = 0.0;  // the most negative term: some rank's pass failed (-1 pipeline, -3 row order)
        for (int q = 0; q < x.world; q++) {
            const unsigned long long* src = exchange_slot(x.peers[x.rank], stride, buf, q) + 2 * i;
            unsigned long long w0, w1;
            for (;;) {
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w0) : "l"(src) : "memory");
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w1) : "l"(src + 1) : "memory");
                if ((w0 & 0xffffffff00000000ULL) == tag && (w1 & 0xffffffff00000000ULL) == tag) break;
                if (timed_out || clock64() - start > x.timeout_cycles) {  // a peer is gone (or very late)
                    timed_out = 1;
                    w0 = w1 = 0ULL;
                    break;
                }
                __nanosleep(32);
            }
            const double term = __longlong_as_double(static_cast<long long>((w0 & 0xffffffffULL) | (w1 << 32)));
            worst = fmin(worst, term);
            s += term;
        }
        if (i < 5) {
            if (i == 4 && worst < 0.0) s = worst > -2.0 ? kBadInputsPipelineTimeout : kBadInputsRowOrder;
            record[i] = s;
        } else {
            global_lengths[i - 5] = s;
            if (x.lengths_out) x.lengths_out[i - 5] = s;
        }
    }
    __syncthreads();
    if (tid < 5) out[tid] = (tid == 4 && timed_out) ? kBadInputsExchangeTimeout : record[tid];  // some rank never answered
    block_weights<kReduceThreads>(global_lengths, x.n_seq, x.reduction, x.length_alpha, x.weights_out, x.meta_out,
                                  scratch);
}

// ---- variant table of the pipelined kernel --------------------------------------------------------
struct Variant {
    int cluster, threads, vec, tj, stages;
    const char* name;
};

// Capacity of a variant in floats: cluster * threads * vec * 4.  Name: cluster x threads x vec.
constexpr Variant kVariants[] = {
    {1, 128, 16, 4, 6, "1x128x16"},   // 0: <=   8192   48 KB ring of 8 KB stages, four CTAs per SM
    {2, 128, 16, 4, 6, "2x128x16"},   // 1: <=  16384
    {4, 128, 16, 4, 6, "4x128x16"},   // 2: <=  32768
    {8, 128, 16, 4, 6, "8x128x16"},   // 3: <=  65536   (GPT-2's 50,304)
    {8, 256, 16, 4, 6, "8x256x16"},   // 4: <= 131072   96 KB ring, two CTAs per SM
    {8, 512, 16, 4, 6, "8x512x16"},   // 5: <= 262144   192 KB ring of 32 KB stages, one CTA per SM
};
constexpr int kNumVariants = sizeof(kVariants) / sizeof(kVariants[0]);

template <int THREADS, int VEC, int TJ, int STAGES, int CLUSTER, int MINB, bool CHECK>
cudaError_t launch_variant(const LogitsArgs& a, cudaStream_t stream) {
    auto kernel = logits_pipelined_kernel<THREADS, VEC, TJ, STAGES, CLUSTER, MINB, CHECK>;
    constexpr size_t ring_bytes = static_cast<size_t>(STAGES) * TJ * THREADS * sizeof(float4);
    // per device: opt in to the large dynamic shared memory and find how many clusters fit at once
    // (two host threads may fill the same entry at once: both compute the same number)
    static std::atomic<int> clusters_cached[64];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = ring_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = CLUSTER > 1 ? 1 : 0;

    int max_clusters = clusters_cached[dev].load(std::memory_order_acquire);
    if (max_clusters == 0) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring_bytes));
        if (err != cudaSuccess) return err;
        int sms = 0;
        err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return err;
        if (CLUSTER == 1) {
            // plain launch: every SM takes CTAs independently
            int per_sm = 0;
            err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, ring_bytes);
            if (err != cudaSuccess) return err;
            max_clusters = per_sm * sms;
        } else {
            cfg.gridDim = dim3(static_cast<unsigned>(sms / CLUSTER * CLUSTER * 4), 1, 1);
            err = cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg);
            if (err != cudaSuccess) return err;
        }
        if (max_clusters < 1) return cudaErrorLaunchOutOfResources;
        clusters_cached[dev].store(max_clusters, std::memory_order_release);
    }
    const long long clusters = a.n_rows < max_clusters ? a.n_rows : max_clusters;
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * CLUSTER), 1, 1);
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <bool CHECK>
cudaError_t launch_by_index(int variant, const LogitsArgs& a, cudaStream_t stream) {
    switch (variant) {
        case 0: return launch_variant<128, 16, 4, 6, 1, 4, CHECK>(a, stream);
        case 1: return launch_variant<128, 16, 4, 6, 2, 4, CHECK>(a, stream);
        case 2: return launch_variant<128, 16, 4, 6, 4, 4, CHECK>(a, stream);
        case 3: return launch_variant<128, 16, 4, 6, 8, 4, CHECK>(a, stream);
        case 4: return launch_variant<256, 16, 4, 6, 8, 2, CHECK>(a, stream);
        case 5: return launch_variant<512, 16, 4, 6, 8, 1, CHECK>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

bool variant_fits(int variant, int P) {
    const Variant& v = kVariants[variant];
    const long long P4 = P >> 2;
    const long long per_cta = (P4 + v.cluster - 1) / v.cluster;
    return per_cta <= static_cast<long long>(v.threads) * v.vec;
}

}  // namespace

// Test and tuning hook (process-wide): -1 restores the dispatcher's own choice.
namespace {
std::atomic<int> g_forced_variant{-1};
}
int set_forced_variant(int variant) {
    if (variant >= kNumVariants) return -1;
    g_forced_variant.store(variant < 0 ? -1 : variant, std::memory_order_relaxed);
    return 0;
}

int resident_variant_count() { return kNumVariants; }

const char* resident_variant_name(int variant) {
    return variant >= 0 && variant < kNumVariants ? kVariants[variant].name : nullptr;
}

// Returns the variant index for this row layout, or -1 when only the streaming kernel applies.
int pick_resident_variant(const void* logits, const void* dlogits, int V, int P, long long n_rows) {
    (void)V;
    (void)n_rows;
    if ((P & 3) != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(logits) & 15u) || (reinterpret_cast<uintptr_t>(dlogits) & 15u)) return -1;
    const int forced = g_forced_variant.load(std::memory_order_relaxed);
    if (forced >= 0 && forced < kNumVariants) return variant_fits(forced, P) ? forced : -1;
    // smallest CTAs whose cluster (at most 8) holds the row: four CTAs per SM overlap one another's serial phases
    for (int idx = 0; idx < kNumVariants; idx++)
        if (variant_fits(idx, P)) return idx;
    return -1;
}

cudaError_t launch_logits_resident(int variant, bool check, const LogitsArgs& a, cudaStream_t stream) {
    return check ? launch_by_index<true>(variant, a, stream) : launch_by_index<false>(variant, a, stream);
}

cudaError_t launch_logits_streaming(bool check, const LogitsArgs& a, cudaStream_t stream) {
    const unsigned blocks = static_cast<unsigned>(a.n_rows);
    if (check)
        logits_streaming_kernel<true><<<blocks, kStreamThreads, 0, stream>>>(a);
    else
        logits_streaming_kernel<false><<<blocks, kStreamThreads, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_logits_reduce(const LogitsArgs& a, const ExchangeArgs& x, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((a.n_rows + kReduceThreads - 1) / kReduceThreads), 1, 1);
    cfg.blockDim = dim3(kReduceThreads, 1, 1);
    cfg.stream = stream;
    // programmatic dependent launch: the blocks may start before the row kernel has drained; the
    // kernel itself waits (griddepcontrol.wait) before touching what the row kernel produced
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, logits_reduce_kernel, a, x);
}

}  // namespace grpo_b200
