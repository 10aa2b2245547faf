// Fused logits path (K2): log-softmax, selected-token gather, token loss and log-softmax
// backward in one pass, writing dL/dlogits over the logits.
//
// Replaces grpo_logits_fused_kernel and the three-kernel "separate" pipeline of the reference
// (src/cuda/grpo_loss_cuda.cu:181-349).  Two kernels live here:
//
//  * the ROW-RESIDENT kernel: a thread-block cluster of CLUSTER CTAs owns one row; every
//    thread keeps VEC float4 chunks of the row in registers, so the row is read from HBM once
//    (128-bit streaming loads), reduced on chip (registers -> warp shuffles -> shared memory
//    -> distributed shared memory across the cluster), and the gradient is written straight
//    from the same registers (128-bit streaming stores).  One exp per element: the thread's
//    e_i = 2^((x_i - m_thread) * log2 e) are kept and rescaled by one per-thread factor
//    once the row maximum and normaliser are known.
//  * the STREAMING kernel: one CTA per row, three sweeps over the row (max, normaliser,
//    gradient; the second and third come from L2 for rows of ordinary size).  It takes any V, P
//    and alignment, and is what GRPO_B200_LOGITS_SEPARATE selects.
//
// Neither kernel touches a masked row's logits or selected id; both write zeros over all P
// columns of a masked row and over columns [V, P) of an active one.  Per-row loss terms go to
// a workspace and are summed in a fixed order by a finalize kernel: no atomics anywhere.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace grpo_b200 {

int g_forced_variant = -1;

namespace {

struct RowStat {
    float m;  // running maximum (-inf when empty)
    float s;  // sum of 2^((x - m) * log2 e) (0 when empty)
};

// Merge of two (max, normaliser) pairs.  Symmetric in its arguments, so a butterfly leaves the
// same bits in every lane.  An empty side (m = -inf, s = 0) contributes exactly 0.
__device__ __forceinline__ RowStat merge(RowStat a, RowStat b) {
    RowStat r;
    r.m = fmaxf(a.m, b.m);
    const float ref = r.m == -CUDART_INF_F ? 0.0f : r.m;
    r.s = a.s * ex2_approx((a.m - ref) * kLog2e) + b.s * ex2_approx((b.m - ref) * kLog2e);
    return r;
}

__device__ __forceinline__ RowStat warp_merge(RowStat v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        RowStat other;
        other.m = __shfl_xor_sync(0xffffffffu, v.m, o);
        other.s = __shfl_xor_sync(0xffffffffu, v.s, o);
        v = merge(v, other);
    }
    return v;
}

// What the row leader hands to every thread of its CTA for the backward sweep.
struct RowBroadcast {
    float row_max;      // M
    float neg_g_over_z; // -dlogp / normaliser (normaliser relative to e^M)
    float g;            // dlogp
    int selected;
};

// 2^(x*log2e - shift) with shift = fl(m*log2e) differs from e^(x-m) by the factor 2^delta,
// delta = m*log2e - shift, which one FMA recovers exactly.  Returns 2^(-delta) (to first order,
// |delta| < 2^-18), the factor that converts such terms to "relative to e^m".
__device__ __forceinline__ float shift_correction(float m_ref, float shift) {
    const float delta = fmaf(m_ref, kLog2e, -shift);
    return fmaf(-delta, 0.69314718f, 1.0f);
}

// Row-level scalar work, done by one thread per CTA: log-sum-exp in double, selected
// log-probability, token loss.  Follows src/cpu/grpo_loss.cpp:214-215 and :137-160.
__device__ __forceinline__ RowBroadcast row_leader(const LogitsArgs& a, long long row, RowStat st, float x_sel,
                                                   int sel, bool bad_input, bool write_terms) {
    const long long seq = (a.row_offset + row) / a.tokens_per_seq;
    const double lse = static_cast<double>(st.m) + log(static_cast<double>(st.s));
    const float lp_new = static_cast<float>(static_cast<double>(x_sel) - lse);
    const float adv = __ldg(a.advantages + seq);
    const float w = __ldg(a.weights + seq);
    const TokenTerms t = token_terms<true>(lp_new, __ldg(a.logp_old + row), __ldg(a.logp_ref + row), adv, w,
                                           a.clip_eps, a.beta);
    RowBroadcast b;
    b.row_max = st.m;
    b.g = t.grad;
    b.neg_g_over_z = -t.grad / st.s;
    b.selected = sel;
    if (write_terms) {
        float flags = 0.0f;
        if (!finite_f(t.grad) || !finite_f(b.neg_g_over_z)) flags += kRowBadGrad;
        if (bad_input) flags += kRowBadInput;
        a.row_terms[row] = make_float4(t.loss, t.pg, t.kl, flags);
        if (a.selected_logp) a.selected_logp[row] = lp_new;
    }
    return b;
}

__device__ __forceinline__ float max4(float4 v) { return fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }

// ---------------------------------------------------------------------------------------------
// Row-resident kernel.  Requires P % 4 == 0 and 16-byte aligned row starts; the dispatcher
// guarantees ceil(P/4 / CLUSTER) <= THREADS * VEC.
// ---------------------------------------------------------------------------------------------
template <int THREADS, int VEC, int CLUSTER, bool CHECK>
__global__ void __launch_bounds__(THREADS) logits_resident_kernel(const LogitsArgs a) {
    constexpr int WARPS = THREADS / 32;
    __shared__ RowStat warp_stat[WARPS];
    __shared__ float warp_chk[WARPS];
    __shared__ float4 exchange;  // this CTA's {m, s, finite-check, 0}, read by its cluster peers
    __shared__ RowBroadcast bc;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const long long row = blockIdx.x / CLUSTER;
    unsigned crank = 0;
    if (CLUSTER > 1) crank = cg::this_cluster().block_rank();

    const int P4 = a.P >> 2;
    const int per_cta = (P4 + CLUSTER - 1) / CLUSTER;
    const int c0 = crank * per_cta;
    const int c1 = min(c0 + per_cta, P4);
    const float4* in = reinterpret_cast<const float4*>(a.logits + row * static_cast<long long>(a.P));
    float4* out = reinterpret_cast<float4*>(a.dlogits + row * static_cast<long long>(a.P));
    const int V = a.V;

    if (a.mask[row] == 0) {  // uniform over the cluster: nobody reaches a cluster barrier
        const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            const int c = c0 + j * THREADS + tid;
            if (c < c1) store_stream(out + c, zero);
        }
        if (crank == 0 && tid == 0) {
            a.row_terms[row] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (a.selected_logp) a.selected_logp[row] = 0.0f;
        }
        return;
    }

    // ---- the selected logit, fetched before anything of the row is overwritten
    int sel = 0;
    float x_sel = 0.0f;
    bool bad_sel = false;
    if (tid == 0) {
        sel = a.selected[row];
        if (sel < 0 || sel >= V) {  // host layer rejects this earlier; never read out of the row
            bad_sel = true;
            sel = 0;
        }
        x_sel = a.logits[row * static_cast<long long>(a.P) + sel];
    }

    // ---- one read of the row: VEC independent 128-bit loads per thread
    float4 x[VEC];
    const float ninf = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        const int c = c0 + j * THREADS + tid;
        if (c < c1 && 4 * c < V)
            x[j] = load_stream(in + c);
        else
            x[j] = make_float4(ninf, ninf, ninf, ninf);
    }
    float chk = 0.0f;
    float m = ninf;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        const int c = c0 + j * THREADS + tid;
        if (4 * c + 4 > V && 4 * c < V) {  // the one chunk that straddles column V: drop the padding
            if (4 * c + 1 >= V) x[j].y = ninf;
            if (4 * c + 2 >= V) x[j].z = ninf;
            if (4 * c + 3 >= V) x[j].w = ninf;
            if (CHECK) {
                chk = fmaf(x[j].x, 0.0f, chk);
                if (4 * c + 1 < V) chk = fmaf(x[j].y, 0.0f, chk);
                if (4 * c + 2 < V) chk = fmaf(x[j].z, 0.0f, chk);
            }
        } else if (CHECK && 4 * c < V && c < c1) {
            // x * 0 is NaN for an infinite or NaN logit and 0 otherwise
            chk = fmaf(x[j].x, 0.0f, chk);
            chk = fmaf(x[j].y, 0.0f, chk);
            chk = fmaf(x[j].z, 0.0f, chk);
            chk = fmaf(x[j].w, 0.0f, chk);
        }
        m = fmaxf(m, max4(x[j]));
    }

    // ---- one exp per element, kept in the registers that held the logits
    const float m_ref = m == ninf ? 0.0f : m;
    const float shift = m_ref * kLog2e;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        x[j].x = ex2_approx(fmaf(x[j].x, kLog2e, -shift));
        x[j].y = ex2_approx(fmaf(x[j].y, kLog2e, -shift));
        x[j].z = ex2_approx(fmaf(x[j].z, kLog2e, -shift));
        x[j].w = ex2_approx(fmaf(x[j].w, kLog2e, -shift));
        s0 += x[j].x;
        s1 += x[j].y;
        s2 += x[j].z;
        s3 += x[j].w;
    }
    RowStat st;
    st.m = m;
    // the thread's terms are relative to 2^shift with shift = fl(m * log2 e); fold the rounding of
    // that product back in so that s is relative to e^m, as merge() assumes
    const float corr = shift_correction(m_ref, shift);
    st.s = ((s0 + s1) + (s2 + s3)) * corr;

    // ---- CTA reduction: shuffles, then one shared-memory round
    st = warp_merge(st);
    if (CHECK) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) chk += __shfl_xor_sync(0xffffffffu, chk, o);
    }
    if (lane == 0) {
        warp_stat[warp] = st;
        if (CHECK) warp_chk[warp] = chk;
    }
    __syncthreads();

    if (warp == 0) {
        RowStat v;
        v.m = ninf;
        v.s = 0.0f;
        float c = 0.0f;
        if (lane < WARPS) {
            v = warp_stat[lane];
            if (CHECK) c = warp_chk[lane];
        }
        v = warp_merge(v);
        if (CHECK) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        }
        if (CLUSTER > 1) {
            if (lane == 0) exchange = make_float4(v.m, v.s, c, 0.0f);
        } else if (lane == 0) {
            bc = row_leader(a, row, v, x_sel, sel, bad_sel || (CHECK && c != 0.0f), true);
        }
    }

    if (CLUSTER > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();  // every CTA's exchange record is visible cluster-wide
        if (warp == 0) {
            RowStat v;
            v.m = ninf;
            v.s = 0.0f;
            float c = 0.0f;
            if (lane < CLUSTER) {
                const float4 e = *cluster.map_shared_rank(&exchange, lane);
                v.m = e.x;
                v.s = e.y;
                c = e.z;
            }
            v = warp_merge(v);
            if (CHECK) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
            }
            // every CTA's leader repeats the same scalar math on the same bits; rank 0 records it
            if (lane == 0) bc = row_leader(a, row, v, x_sel, sel, bad_sel || (CHECK && c != 0.0f), crank == 0);
        }
        cluster.barrier_arrive();  // peers may retire once everyone has read their records
    }
    __syncthreads();

    // ---- backward sweep from registers: g * (onehot - p) = e_i * coef + [i == sel] * g
    const RowBroadcast b = bc;
    const float coef = ex2_approx((m_ref - b.row_max) * kLog2e) * corr * b.neg_g_over_z;
    const int sel_chunk = b.selected >> 2, sel_lane = b.selected & 3;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        const int c = c0 + j * THREADS + tid;
        if (c < c1) {
            float4 o;
            if (4 * c < V) {
                o.x = x[j].x * coef;
                o.y = x[j].y * coef;
                o.z = x[j].z * coef;
                o.w = x[j].w * coef;
                if (c == sel_chunk) {
                    if (sel_lane == 0) o.x += b.g;
                    if (sel_lane == 1) o.y += b.g;
                    if (sel_lane == 2) o.z += b.g;
                    if (sel_lane == 3) o.w += b.g;
                }
                if (4 * c + 4 > V) {  // padding columns inside the straddling chunk
                    if (4 * c + 1 >= V) o.y = 0.0f;
                    if (4 * c + 2 >= V) o.z = 0.0f;
                    if (4 * c + 3 >= V) o.w = 0.0f;
                }
            } else {
                o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
            store_stream(out + c, o);
        }
    }
    if (CLUSTER > 1) cg::this_cluster().barrier_wait();
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
    __shared__ RowBroadcast bc;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long row = blockIdx.x;
    const float* in = a.logits + row * static_cast<long long>(a.P);
    float* out = a.dlogits + row * static_cast<long long>(a.P);
    const int V = a.V, P = a.P;

    if (a.mask[row] == 0) {
        for (int v = tid; v < P; v += kStreamThreads) out[v] = 0.0f;
        if (tid == 0) {
            a.row_terms[row] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (a.selected_logp) a.selected_logp[row] = 0.0f;
        }
        return;
    }

    // sweep 1: maximum (and the finiteness probe)
    float m = -CUDART_INF_F, chk = 0.0f;
    for (int v = tid; v < V; v += kStreamThreads) {
        const float x = in[v];
        m = fmaxf(m, x);
        if (CHECK) chk = fmaf(x, 0.0f, chk);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (CHECK) chk += __shfl_xor_sync(0xffffffffu, chk, o);
    }
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
    __syncthreads();

    // sweep 2: normaliser relative to the row maximum
    const float shift = m * kLog2e;
    float s = 0.0f;
    for (int v = tid; v < V; v += kStreamThreads) s += ex2_approx(fmaf(in[v], kLog2e, -shift));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (tid == 0) {
        float z = 0.0f;
#pragma unroll
        for (int k = 0; k < WARPS; k++) z += red[k];
        int sel = a.selected[row];
        bool bad = CHECK && chk != 0.0f;
        if (sel < 0 || sel >= V) {
            bad = true;
            sel = 0;
        }
        RowStat st;
        st.m = m;
        st.s = z * shift_correction(m, shift);
        bc = row_leader(a, row, st, in[sel], sel, bad, true);
    }
    __syncthreads();

    // sweep 3: gradient; each element is read and then overwritten by the same thread
    const RowBroadcast b = bc;
    const float coef = b.neg_g_over_z * shift_correction(m, shift);
    for (int v = tid; v < V; v += kStreamThreads) {
        const float e = ex2_approx(fmaf(in[v], kLog2e, -shift));
        out[v] = e * coef + (v == b.selected ? b.g : 0.0f);
    }
    for (int v = V + tid; v < P; v += kStreamThreads) out[v] = 0.0f;
}

// One block sums the per-row terms in a fixed order (double accumulators).
__global__ void __launch_bounds__(1024) logits_finalize_kernel(const float4* __restrict__ terms, long long n_rows,
                                                               grpo_b200_result_t* result) {
    __shared__ double scratch[5 * 1024 / 32];
    double v[5] = {0.0, 0.0, 0.0, 0.0, 0.0};
    for (long long r = threadIdx.x; r < n_rows; r += 1024) {
        const float4 t = terms[r];
        v[0] += static_cast<double>(t.x);
        v[1] += static_cast<double>(t.y);
        v[2] += static_cast<double>(t.z);
        const int flags = static_cast<int>(t.w);
        v[3] += (flags & 1) ? 1.0 : 0.0;
        v[4] += (flags & 2) ? 1.0 : 0.0;
    }
    block_sum<1024, 5>(v, scratch);
    if (threadIdx.x == 0) {
        result->loss = v[0];
        result->pg_loss = v[1];
        result->kl = v[2];
        result->bad_grads = v[3];
        result->bad_inputs = v[4];
    }
}

// ---- variant table of the row-resident kernel ---------------------------------------------------
struct Variant {
    int cluster, threads, vec;
    const char* name;
};

// Capacity of a variant in floats: cluster * threads * vec * 4.
constexpr Variant kVariants[] = {
    {1, 256, 8, "1x256x8"},    // 0:  <=   8192
    {2, 256, 8, "2x256x8"},    // 1:  <=  16384
    {4, 256, 8, "4x256x8"},    // 2:  <=  32768
    {8, 256, 8, "8x256x8"},    // 3:  <=  65536
    {8, 512, 8, "8x512x8"},    // 4:  <= 131072
    {16, 256, 8, "16x256x8"},  // 5:  <= 131072 (non-portable cluster size)
    {2, 512, 8, "2x512x8"},    // 6:  <=  32768
    {1, 1024, 8, "1x1024x8"},  // 7:  <=  32768
    {4, 512, 8, "4x512x8"},    // 8:  <=  65536
    {2, 1024, 8, "2x1024x8"},  // 9:  <=  65536
    {4, 1024, 8, "4x1024x8"},  // 10: <= 131072
    {8, 128, 8, "8x128x8"},    // 11: <=  32768
    {8, 256, 4, "8x256x4"},    // 12: <=  32768
    {16, 256, 4, "16x256x4"},  // 13: <=  65536
    {4, 512, 4, "4x512x4"},    // 14: <=  32768
    {1, 128, 2, "1x128x2"},    // 15: <=   1024
    {16, 512, 4, "16x512x4"},  // 16: <= 131072
};
constexpr int kNumVariants = sizeof(kVariants) / sizeof(kVariants[0]);

template <int THREADS, int VEC, int CLUSTER, bool CHECK>
cudaError_t launch_variant(const LogitsArgs& a, cudaStream_t stream) {
    auto kernel = logits_resident_kernel<THREADS, VEC, CLUSTER, CHECK>;
    if (CLUSTER > 8) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (err != cudaSuccess) return err;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(a.n_rows * CLUSTER), 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = CLUSTER > 1 ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <bool CHECK>
cudaError_t launch_by_index(int variant, const LogitsArgs& a, cudaStream_t stream) {
    switch (variant) {
        case 0: return launch_variant<256, 8, 1, CHECK>(a, stream);
        case 1: return launch_variant<256, 8, 2, CHECK>(a, stream);
        case 2: return launch_variant<256, 8, 4, CHECK>(a, stream);
        case 3: return launch_variant<256, 8, 8, CHECK>(a, stream);
        case 4: return launch_variant<512, 8, 8, CHECK>(a, stream);
        case 5: return launch_variant<256, 8, 16, CHECK>(a, stream);
        case 6: return launch_variant<512, 8, 2, CHECK>(a, stream);
        case 7: return launch_variant<1024, 8, 1, CHECK>(a, stream);
        case 8: return launch_variant<512, 8, 4, CHECK>(a, stream);
        case 9: return launch_variant<1024, 8, 2, CHECK>(a, stream);
        case 10: return launch_variant<1024, 8, 4, CHECK>(a, stream);
        case 11: return launch_variant<128, 8, 8, CHECK>(a, stream);
        case 12: return launch_variant<256, 4, 8, CHECK>(a, stream);
        case 13: return launch_variant<256, 4, 16, CHECK>(a, stream);
        case 14: return launch_variant<512, 4, 4, CHECK>(a, stream);
        case 15: return launch_variant<128, 2, 1, CHECK>(a, stream);
        case 16: return launch_variant<512, 4, 16, CHECK>(a, stream);
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

int resident_variant_count() { return kNumVariants; }

const char* resident_variant_name(int variant) {
    return variant >= 0 && variant < kNumVariants ? kVariants[variant].name : nullptr;
}

// Returns the variant index for this row layout, or -1 when only the streaming kernel applies.
int pick_resident_variant(const void* logits, const void* dlogits, int V, int P) {
    (void)V;
    if ((P & 3) != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(logits) & 15u) || (reinterpret_cast<uintptr_t>(dlogits) & 15u)) return -1;
    if (g_forced_variant >= 0 && g_forced_variant < kNumVariants)
        return variant_fits(g_forced_variant, P) ? g_forced_variant : -1;
    // smallest cluster that holds the row with 256-thread CTAs of 8 chunks per thread
    static const int order[] = {15, 0, 1, 2, 3, 4};
    for (int idx : order)
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

cudaError_t launch_logits_finalize(const LogitsArgs& a, cudaStream_t stream) {
    logits_finalize_kernel<<<1, 1024, 0, stream>>>(a.row_terms, a.n_rows, a.result);
    return cudaGetLastError();
}

}  // namespace grpo_b200
