// Row softmax with a per-row valid length (causal attention scores, router logits).
//
// Reference: the softmax step of `attention_into` (src/model/llama/cpu_path.rs:175-183):
//   max = fold(-inf, f32::max) over s[0..n) ; s = exp(s - max) ; sum = sum(s) ; s = s / sum
// with n = pos + 1: causality is a row LENGTH, entries past n are never touched.  Here
// those entries of the output are written as 0 so the full [n_rows, row_len] matrix is
// defined.  GPU twin: `attention_softmax` (src/ops/kernels_wgpu.rs:795-864).
//
// Bound by HBM: reads only the valid prefix of each row, writes the full row, the row
// stays in registers between the three passes (max, exp+sum, divide).
//   - rows up to 1024 entries: one warp per row, statistics by warp shuffles only;
//   - rows up to 32768 entries: one CTA per row, shuffles + a shared-memory combine;
//   - anything else (odd lengths, unaligned, longer): three passes over global memory.
#include <math.h>

#include <cooperative_groups.h>

#include "agn_common.cuh"

namespace cg = cooperative_groups;

namespace {

struct SoftmaxArgs {
    const float *in;
    void *out;  // probabilities: float, or __half / __nv_bfloat16 (the kernels' template parameter OT)
    const int32_t *n_valid;
    float *sums;  // non-null: store the unnormalised exp(s - max) and the row sums (the reference's GPU form)
    int64_t n_rows, row_len, row_stride;
    int causal_period, causal_offset;
    int leave_tail;  // 1: entries past the valid length are not written (the reference's behaviour); 0: written as 0
    float scale;     // scores are multiplied by this (> 0) before the softmax; 1 for the plain form
    float exp_coef;  // scale * log2(e): exp(scale * (s - max)) = 2^((s - max) * exp_coef)
};

__device__ __forceinline__ int64_t valid_len(const SoftmaxArgs &a, int64_t r) {
    int64_t nv;
    if (a.n_valid) nv = a.n_valid[r];
    // (row numbers fit 31 bits — the host checks — so the remainder is a 32-bit one: a 64-bit
    // remainder is ~100 instructions in every thread of kernels that run ~600 per thread)
    else if (a.causal_period > 0) nv = (int64_t)a.causal_offset + (int64_t)((uint32_t)r % (uint32_t)a.causal_period) + 1;
    else nv = a.row_len;
    if (nv > a.row_len) nv = a.row_len;
    if (nv < 0) nv = 0;
    return nv;
}


// Float4 number i of a row whose first nv entries are valid.  The load is one predicated
// instruction (so that a thread's loads are all issued back to back); mask_tail then sets
// the invalid entries to -inf, and only the one float4 that straddles nv pays for it.
__device__ __forceinline__ float4 load_valid(const float4 *row, int i, int nv) {
    return 4 * i < nv ? agn_ld_stream(row + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
}
__device__ __forceinline__ void mask_tail(float4 &v, int i, int nv) {
    const int e = 4 * i;
    if (e < nv && e + 3 >= nv) {
        if (e + 1 >= nv) v.y = -INFINITY;
        if (e + 2 >= nv) v.z = -INFINITY;
        v.w = -INFINITY;
    }
}

// Entries past the valid length are defined as 0 whatever the row holds (a NaN or an infinity in
// the row makes the factor NaN, and 0 * NaN would leak into the straddling float4).
__device__ __forceinline__ void zero_tail(float4 &v, int i, int nv) {
    const int e = 4 * i;
    if (e < nv && e + 3 >= nv) {
        if (e + 1 >= nv) v.y = 0.0f;
        if (e + 2 >= nv) v.z = 0.0f;
        v.w = 0.0f;
    }
}

// Stores float4 number i of an output row.  leave_tail = false: entries past the valid length are
// written as 0.  leave_tail = true: they are not written at all, which is what the reference's loop
// over `scores[..seq_len]` does (src/model/llama/cpu_path.rs:168-183) and saves a third of a causal
// softmax's traffic; the float4 that straddles the valid length is then stored entry by entry.
template <typename OT>
__device__ __forceinline__ void store_probs(OT *out, int i, float4 o, int nv, int n4, bool leave_tail) {
    if (i >= n4) return;
    const int e = 4 * i;
    if (e + 3 < nv) {  // wholly valid: the common case, nothing to mask
        ActVec<OT>::store(out, i, o);
    } else if (!leave_tail) {  // straddles the valid length (or lies past it, with o = 0): zeros behind it
        zero_tail(o, i, nv);
        ActVec<OT>::store(out, i, o);
    } else if (e < nv) {  // one to three valid entries, the rest left untouched
        ActVec<OT>::store1(out, e, o.x);
        if (e + 1 < nv) ActVec<OT>::store1(out, e + 1, o.y);
        if (e + 2 < nv) ActVec<OT>::store1(out, e + 2, o.z);
    }
}

// Float4 number i of an output row when it lies wholly past the valid length: zeros, or nothing.
template <typename OT>
__device__ __forceinline__ void store_past_valid(OT *out, int i, int n4, bool leave_tail) {
    if (!leave_tail && i < n4) ActVec<OT>::store(out, i, make_float4(0.f, 0.f, 0.f, 0.f));
}

// exp(v - m) as 2^((v - m) * log2 e) with the hardware ex2: three instructions per element
// instead of the ~10 of expf, which made these kernels issue-bound (84 % issue-active at
// 59 % of DRAM peak).  Arguments are <= 0, so the result is in [0, 1] and its absolute
// error (~2^-22 + |v - m| * 2^-24 relative) stays far below 1e-5 of the row scale.  A masked
// entry (-inf) gives exactly 0, so no per-element predicate is needed.
// A positive score scale folds into the coefficient: max(scale * s) = scale * max(s).
__device__ __forceinline__ float exp_shifted(float v, float m, float coef) {
    float r;
    const float t = (v - m) * coef;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
    return r;
}
__device__ __forceinline__ float ex2_approx(float t) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
    return r;
}
// Four at a time.  The subtraction, the multiplication, the row sum and the final scaling run on
// Blackwell's packed f32x2 instructions (two IEEE round-to-nearest results per instruction, the
// same bits as the scalar operations): these kernels are bound by instruction issue once the
// output shrinks, and this takes a third of the floating-point instructions out.
__device__ __forceinline__ float4 exp4(float4 v, float m, float coef) {
    const float2 nm = make_float2(-m, -m), cc = make_float2(coef, coef);
    const float2 lo = __fmul2_rn(__fadd2_rn(make_float2(v.x, v.y), nm), cc);
    const float2 hi = __fmul2_rn(__fadd2_rn(make_float2(v.z, v.w), nm), cc);
    return make_float4(ex2_approx(lo.x), ex2_approx(lo.y), ex2_approx(hi.x), ex2_approx(hi.y));
}
__device__ __forceinline__ float hsum4(float4 v) {  // (x + y) + (z + w)
    const float2 p = __fadd2_rn(make_float2(v.x, v.z), make_float2(v.y, v.w));
    return p.x + p.y;
}
__device__ __forceinline__ float4 scale4(float4 v, float f) {
    const float2 ff = make_float2(f, f);
    const float2 lo = __fmul2_rn(make_float2(v.x, v.y), ff), hi = __fmul2_rn(make_float2(v.z, v.w), ff);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Very short rows (router logits, <= 32 entries): one thread per row, everything in registers.
template <typename OT, int VPT>
__global__ void __launch_bounds__(256)
softmax_thread_rows_kernel(const SoftmaxArgs a) {
    agn_pdl_prologue();
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= a.n_rows) return;
    const int nv = (int)valid_len(a, r);
    const int n4 = (int)(a.row_len >> 2);
    const float4 *in = reinterpret_cast<const float4 *>(a.in + r * a.row_stride);
    OT *out = static_cast<OT *>(a.out) + r * a.row_stride;
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) v[k] = k < n4 ? load_valid(in, k, nv) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
    for (int k = 0; k < VPT; k++) mask_tail(v[k], k, nv);
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT; k++) m = agn_max_acc4(m, v[k]);
    float sum = 0.0f;
    if (nv > 0) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            v[k] = exp4(v[k], m, a.exp_coef);
            sum += hsum4(v[k]);
        }
    }
    if (a.sums) a.sums[r] = sum;
    const float inv = (a.sums || nv <= 0) ? 1.0f : 1.0f / sum;
#pragma unroll
    for (int k = 0; k < VPT; k++)
        {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (4 * k < nv) o = scale4(v[k], inv);
            store_probs<OT>(out, k, o, nv, n4, a.leave_tail != 0);
        }
}

template <typename OT, int VPL>
__global__ void __launch_bounds__(256, VPL >= 16 ? 2 : 4)
softmax_warp_rows_kernel(const SoftmaxArgs a) {
    agn_pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= a.n_rows) return;  // whole warp leaves together
    const int nv = (int)valid_len(a, r);
    const int n4 = (int)(a.row_len >> 2);
    const float4 *in = reinterpret_cast<const float4 *>(a.in + r * a.row_stride);
    OT *out = static_cast<OT *>(a.out) + r * a.row_stride;
    float4 v[VPL];
#pragma unroll
    for (int k = 0; k < VPL; k++) v[k] = load_valid(in, lane + 32 * k, nv);
#pragma unroll
    for (int k = 0; k < VPL; k++) mask_tail(v[k], lane + 32 * k, nv);
    // float4 that lie wholly past the valid length (half of a causal matrix) cost nothing below:
    // for k >= 1 a whole warp is on the same side of the boundary, so the branches are uniform
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPL; k++)
        if (4 * (lane + 32 * k) < nv) m = agn_max_acc4(m, v[k]);
    m = agn_warp_max(m);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < VPL; k++) {
        if (4 * (lane + 32 * k) < nv) {
            v[k] = exp4(v[k], m, a.exp_coef);
            sum += hsum4(v[k]);
        }
    }
    sum = agn_warp_sum(sum);
    if (a.sums && lane == 0) a.sums[r] = sum;
    const float inv = (a.sums || nv <= 0) ? 1.0f : 1.0f / sum;  // s / sum of the CPU path as s * (1/sum): <= 1 ulp apart
#pragma unroll
    for (int k = 0; k < VPL; k++) {
        const int i = lane + 32 * k;
        if (4 * i < nv) store_probs<OT>(out, i, scale4(v[k], inv), nv, n4, a.leave_tail != 0);
        else store_past_valid<OT>(out, i, n4, a.leave_tail != 0);
    }
}

template <typename OT, int VPT>
__global__ void __launch_bounds__(1024)
softmax_block_rows_kernel(const SoftmaxArgs a) {
    agn_pdl_prologue();
    __shared__ float red[32], red_sum[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int64_t r = blockIdx.x;
    const int nv = (int)valid_len(a, r);
    const int n4 = (int)(a.row_len >> 2);
    const float4 *in = reinterpret_cast<const float4 *>(a.in + r * a.row_stride);
    OT *out = static_cast<OT *>(a.out) + r * a.row_stride;
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) v[k] = load_valid(in, threadIdx.x + k * blockDim.x, nv);
#pragma unroll
    for (int k = 0; k < VPT; k++) mask_tail(v[k], threadIdx.x + k * blockDim.x, nv);
    // float4 that lie wholly past the valid length (half of a causal matrix) cost nothing below:
    // a whole warp is on the same side of the boundary except for one, so the branches are uniform
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT; k++)
        if (4 * (threadIdx.x + k * blockDim.x) < nv) m = agn_max_acc4(m, v[k]);
    m = agn_warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < nwarps; w++) m = fmaxf(m, red[w]);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        if (4 * (threadIdx.x + k * blockDim.x) < nv) {
            v[k] = exp4(v[k], m, a.exp_coef);
            sum += hsum4(v[k]);
        }
    }
    sum = agn_warp_sum(sum);
    if (lane == 0) red_sum[warp] = sum;  // (its own array: no barrier between reading the maxima and writing the sums)
    __syncthreads();
    sum = 0.0f;
    for (int w = 0; w < nwarps; w++) sum += red_sum[w];
    if (a.sums && threadIdx.x == 0) a.sums[r] = sum;
    const float inv = (a.sums || nv <= 0) ? 1.0f : 1.0f / sum;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (4 * i < nv) store_probs<OT>(out, i, scale4(v[k], inv), nv, n4, a.leave_tail != 0);
        else store_past_valid<OT>(out, i, n4, a.leave_tail != 0);
    }
}

// Square causal matrices ([heads, L, L], row i of a head has i + 1 valid entries): rows i and
// L-1-i of a head are done by ONE CTA, so every CTA loads and stores the same L + 1 valid entries
// whatever i is.  With a CTA per row, half of the CTAs hold mostly masked rows: their threads keep
// their registers but have no load in flight, and the kernel ends up bound by latency rather than by
// HBM once the output shrinks (16-bit probabilities, or the tail left unwritten).  The CTA's
// threads walk the concatenation [valid part of row A | valid part of row B] in float4 steps;
// maxima and sums are kept per row (two values through every reduction).
template <typename OT, int VPT>
__global__ void __launch_bounds__(1024)
softmax_causal_pair_kernel(const SoftmaxArgs a) {
    agn_pdl_prologue();
    __shared__ float red[2][32], red_sum[2][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int L = (int)a.row_len, n4 = L >> 2;
    const int half_rows = (L + 1) >> 1;
    const uint32_t head_u = blockIdx.x / (uint32_t)half_rows;  // 32-bit division: the grid fits 31 bits
    const int64_t head = head_u;
    const int p = (int)(blockIdx.x - head_u * (uint32_t)half_rows);
    const int rowA = p, rowB = L - 1 - p;       // rowB == rowA for the middle row of an odd L
    const bool twoRows = rowB != rowA;
    const int nvA = rowA + 1, nvB = twoRows ? rowB + 1 : 0;
    const int vA = (nvA + 3) >> 2, vB = (nvB + 3) >> 2;  // float4 that hold valid entries
    const int64_t rA = head * L + rowA, rB = head * L + rowB;
    const float4 *inA = reinterpret_cast<const float4 *>(a.in + rA * a.row_stride);
    const float4 *inB = reinterpret_cast<const float4 *>(a.in + rB * a.row_stride);
    OT *outA = static_cast<OT *>(a.out) + rA * a.row_stride, *outB = static_cast<OT *>(a.out) + rB * a.row_stride;
    // vector j of the concatenation: row A's float4 number j for j < vA, else row B's number j - vA
    float4 v[VPT];
    int idx[VPT];  // float4 index inside its row, or -1; bit 30 set = row B
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int j = threadIdx.x + k * blockDim.x;
        const bool isB = j >= vA;
        const int i = isB ? j - vA : j;
        const bool on = isB ? i < vB : true;
        idx[k] = on ? (i | (isB ? (1 << 30) : 0)) : -1;
        v[k] = on ? agn_ld_stream((isB ? inB : inA) + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    float mA = -INFINITY, mB = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        if (idx[k] >= 0) {
            const bool isB = (idx[k] >> 30) & 1;
            mask_tail(v[k], idx[k] & 0x3fffffff, isB ? nvB : nvA);
            if (isB) mB = agn_max_acc4(mB, v[k]);
            else mA = agn_max_acc4(mA, v[k]);
        }
    }
    mA = agn_warp_max(mA);
    mB = agn_warp_max(mB);
    if (lane == 0) { red[0][warp] = mA; red[1][warp] = mB; }
    __syncthreads();
    mA = -INFINITY; mB = -INFINITY;
    for (int w = 0; w < nwarps; w++) { mA = fmaxf(mA, red[0][w]); mB = fmaxf(mB, red[1][w]); }
    float sA = 0.0f, sB = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        if (idx[k] >= 0) {
            const bool isB = (idx[k] >> 30) & 1;
            v[k] = exp4(v[k], isB ? mB : mA, a.exp_coef);
            const float t = hsum4(v[k]);
            if (isB) sB += t;
            else sA += t;
        }
    }
    sA = agn_warp_sum(sA);
    sB = agn_warp_sum(sB);
    if (lane == 0) { red_sum[0][warp] = sA; red_sum[1][warp] = sB; }  // (own arrays: no barrier between maxima and sums)
    __syncthreads();
    sA = 0.0f; sB = 0.0f;
    for (int w = 0; w < nwarps; w++) { sA += red_sum[0][w]; sB += red_sum[1][w]; }
    if (a.sums && threadIdx.x == 0) {
        a.sums[rA] = sA;
        if (twoRows) a.sums[rB] = sB;
    }
    const float invA = a.sums ? 1.0f : 1.0f / sA, invB = (a.sums || !twoRows) ? 1.0f : 1.0f / sB;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        if (idx[k] >= 0) {
            const bool isB = (idx[k] >> 30) & 1;
            const float inv = isB ? invB : invA;
            store_probs<OT>(isB ? outB : outA, idx[k] & 0x3fffffff, scale4(v[k], inv),
                            isB ? nvB : nvA, n4, a.leave_tail != 0);
        }
    }
    if (!a.leave_tail) {
        // the float4 wholly past the valid length of either row: n4 - vA of row A, then n4 - vB of row B
        const int zA = n4 - vA, zB = twoRows ? n4 - vB : 0;
        for (int z = threadIdx.x; z < zA + zB; z += blockDim.x) {
            if (z < zA) ActVec<OT>::store(outA, vA + z, make_float4(0.f, 0.f, 0.f, 0.f));
            else ActVec<OT>::store(outB, vB + (z - zA), make_float4(0.f, 0.f, 0.f, 0.f));
        }
    }
}

// Persistent form of the CTA-per-row kernel for large batches of rows of 1K-32K entries.  A softmax
// row goes through two block-wide reductions between its loads and its stores, so a CTA that owns
// one row has nothing in flight for most of its life; with causal rows, whose valid part is half
// the row on average, the registers that could hold loads sit idle and the kernel is bound by
// latency (5.0 TB/s when the tail is not written) although HBM has room.  Here a CTA loops over
// rows blockIdx.x, blockIdx.x + gridDim.x, ... and the valid prefixes of its next rows are already
// on their way into a ring of shared-memory slots (one bulk asynchronous copy per row, issued by
// one thread, completing on the slot's mbarrier with a bounded wait), so loads overlap the
// reductions and the stores of the rows before them.
template <typename OT, int VPT>
__global__ void __launch_bounds__(1024)
softmax_ring_kernel(const SoftmaxArgs a, int slots, int slot_bytes, int spin_limit, uint32_t *flags) {
    extern __shared__ __align__(128) unsigned char sm_ring[];
    __shared__ float red[2][32];
    uint64_t *full = reinterpret_cast<uint64_t *>(sm_ring + (size_t)slots * slot_bytes);
    if (threadIdx.x == 0) {
        for (int s = 0; s < slots; s++) agn_mbar_init(&full[s], 1);
        agn_mbar_init_fence();
    }
    __syncthreads();
    agn_pdl_launch_dependents();
    agn_pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n4 = (int)(a.row_len >> 2);
    const int64_t first = blockIdx.x, stride = gridDim.x;
    const int n_my = first < a.n_rows ? (int)((a.n_rows - first + stride - 1) / stride) : 0;
    auto issue = [&](int j) {  // thread 0 only; a row without valid entries brings nothing
        const int64_t r = first + (int64_t)j * stride;
        const int nv = (int)valid_len(a, r);
        if (nv <= 0) return;
        const uint32_t bytes = (uint32_t)((nv + 3) >> 2) * 16u;
        uint64_t *bar = &full[j % slots];
        agn_mbar_expect_tx(bar, bytes);
        agn_bulk_g2s(sm_ring + (size_t)(j % slots) * slot_bytes, a.in + r * a.row_stride, bytes, bar);
    };
    if (threadIdx.x == 0)
        for (int j = 0; j < slots && j < n_my; j++) issue(j);
    uint32_t phase_bits = 0;  // bit s: parity the next wait on slot s expects (flips only when a copy was issued)
    for (int it = 0; it < n_my; it++) {
        const int slot = it % slots;
        const int64_t r = first + (int64_t)it * stride;
        const int nv = (int)valid_len(a, r);
        OT *out = static_cast<OT *>(a.out) + r * a.row_stride;
        int failed = 0;
        if (nv > 0) {
            failed = !agn_mbar_wait(&full[slot], (phase_bits >> slot) & 1u, spin_limit);
            phase_bits ^= 1u << slot;
        }
        const float4 *row = reinterpret_cast<const float4 *>(sm_ring + (size_t)slot * slot_bytes);
        float4 v[VPT];
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            v[k] = (4 * i < nv && !failed) ? row[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
        float m = -INFINITY;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (4 * i < nv) {
                mask_tail(v[k], i, nv);
                m = agn_max_acc4(m, v[k]);
            }
        }
        m = agn_warp_max(m);
        if (lane == 0) red[0][warp] = m;
        // maxima visible; every thread has read its part of the slot; one CTA-wide answer to "did
        // any thread's wait run out", so that all threads leave together
        if (__syncthreads_or(failed)) {
            if (threadIdx.x == 0) {
                atomicOr(flags, AGN_FLAG_TIMEOUT);
                // copies still in flight target this CTA's shared memory: one more bounded wait each
                for (int j = it; j < n_my && j < it + slots; j++) {
                    if ((int)valid_len(a, first + (int64_t)j * stride) <= 0) continue;
                    const uint32_t par = ((phase_bits >> (j % slots)) & 1u) ^ (j == it ? 1u : 0u);
                    (void)agn_mbar_wait(&full[j % slots], par, spin_limit);
                }
            }
            return;
        }
        if (threadIdx.x == 0 && it + slots < n_my) issue(it + slots);
        m = -INFINITY;
        for (int w = 0; w < nwarps; w++) m = fmaxf(m, red[0][w]);
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            if (4 * (threadIdx.x + k * blockDim.x) < nv) {
                v[k] = exp4(v[k], m, a.exp_coef);
                sum += hsum4(v[k]);
            }
        }
        sum = agn_warp_sum(sum);
        if (lane == 0) red[1][warp] = sum;
        __syncthreads();
        sum = 0.0f;
        for (int w = 0; w < nwarps; w++) sum += red[1][w];
        if (a.sums && threadIdx.x == 0) a.sums[r] = sum;
        const float inv = (a.sums || nv <= 0) ? 1.0f : 1.0f / sum;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (4 * i < nv) store_probs<OT>(out, i, scale4(v[k], inv), nv, n4, a.leave_tail != 0);
            else store_past_valid<OT>(out, i, n4, a.leave_tail != 0);
        }
    }
}

// Long rows (8K-64K entries): one thread-block CLUSTER per row.  Each of the C CTAs (256 threads,
// 8 float4 per thread) owns 8192 consecutive entries in registers; the row maximum and the row
// sum are combined across the cluster through distributed shared memory (each CTA publishes its
// partial in its own shared memory, every CTA reads all C partials in rank order after a cluster
// barrier, so all CTAs compute the same value).  Each CTA finishes its own part first (maximum
// m_c, e = exp(v - m_c), sum s_c) and the parts are merged afterwards (M = max m_c,
// S = sum s_c exp(m_c - M), entry = e exp(m_c - M) / S), so one cluster barrier is enough.
// Against one 1024-thread CTA per row this keeps several independent CTAs resident per SM, so
// the loads of one row overlap the exponentials and stores of another.  Cluster barriers are
// hardware barriers: no spin-waits.
template <typename OT, int VPT>
__global__ void __launch_bounds__(512)
softmax_cluster_rows_kernel(const SoftmaxArgs a, int cluster_size) {
    agn_pdl_prologue();
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red[16];
    __shared__ float xch[2];  // this CTA's partial maximum and partial sum, read by its peers
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int rank = (int)cluster.block_rank();
    const int64_t r = blockIdx.x / cluster_size;
    const int nv = (int)valid_len(a, r);
    const int n4 = (int)(a.row_len >> 2);
    const float4 *in = reinterpret_cast<const float4 *>(a.in + r * a.row_stride);
    OT *out = static_cast<OT *>(a.out) + r * a.row_stride;
    // tiles of blockDim float4 are dealt round-robin to the CTAs of the cluster, so the valid prefix
    // of a causal row is spread evenly over them
    const int base = rank * blockDim.x + threadIdx.x, step = cluster_size * blockDim.x;
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) v[k] = load_valid(in, base + k * step, nv);
#pragma unroll
    for (int k = 0; k < VPT; k++) mask_tail(v[k], base + k * step, nv);
    // this CTA's part on its own: maximum m_c, then e = exp(v - m_c) and their sum s_c
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT; k++) m = agn_max_acc4(m, v[k]);
    m = agn_warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nwarps; w++) m = fmaxf(m, red[w]);
    __syncthreads();
    const float m_c = m == -INFINITY ? 0.0f : m;  // a part with no valid entry: every e is exp(-inf) = 0
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        v[k] = exp4(v[k], m_c, a.exp_coef);
        sum += hsum4(v[k]);
    }
    sum = agn_warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < nwarps; w++) t += red[w];
        xch[0] = m;
        xch[1] = t;
    }
    cluster.sync();
    // combine the parts in rank order (the same value in every CTA):
    // M = max m_c, S = sum s_c * exp(m_c - M); this CTA's entries are e * exp(m_c - M) / S
    float M = -INFINITY;
    for (int c = 0; c < cluster_size; c++) M = fmaxf(M, *cluster.map_shared_rank(&xch[0], c));
    float S = 0.0f;
    for (int c = 0; c < cluster_size; c++) {
        const float mc = *cluster.map_shared_rank(&xch[0], c), sc = *cluster.map_shared_rank(&xch[1], c);
        if (mc != -INFINITY) S += sc * exp_shifted(mc, M, a.exp_coef);
    }
    // arrive now, wait before leaving: no CTA may exit (and give up its shared memory) while a
    // peer still reads it, but the stores below need not wait for that
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    if (a.sums && rank == 0 && threadIdx.x == 0) a.sums[r] = S;
    float f = 0.0f;
    if (nv > 0 && m != -INFINITY) f = exp_shifted(m, M, a.exp_coef) * (a.sums ? 1.0f : 1.0f / S);
    // a row whose valid entries are all -inf: exp(-inf - -inf) is NaN in the reference's loop and
    // in the one-CTA kernels; give the same answer here
    if (nv > 0 && M == -INFINITY) f = __int_as_float(0x7fc00000);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int i = base + k * step;
        {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (4 * i < nv) o = scale4(v[k], f);
            store_probs<OT>(out, i, o, nv, n4, a.leave_tail != 0);
        }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <typename OT>
__global__ void __launch_bounds__(256)
softmax_generic_rows_kernel(const SoftmaxArgs a) {
    agn_pdl_prologue();
    __shared__ float red[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int64_t r = blockIdx.x;
    const int64_t nv = valid_len(a, r);
    const float *in = a.in + r * a.row_stride;
    OT *out = static_cast<OT *>(a.out) + r * a.row_stride;
    constexpr bool F32_OUT = sizeof(OT) == 4;
    float m = -INFINITY;
    for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) m = fmaxf(m, in[i]);
    m = agn_warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < nwarps; w++) m = fmaxf(m, red[w]);
    __syncthreads();
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
        const float e = expf((in[i] - m) * a.scale);
        // f32 output: park e in the output row (in may alias out: element i is only ever touched
        // by this thread); a 16-bit output row cannot hold it without rounding, so the last pass
        // evaluates the exponential again
        if (F32_OUT) ActVec<OT>::store1(out, i, e);
        sum += e;
    }
    sum = agn_warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.0f;
    for (int w = 0; w < nwarps; w++) sum += red[w];
    if (a.sums && threadIdx.x == 0) a.sums[r] = sum;
    const float inv = (a.sums || nv <= 0) ? 1.0f : 1.0f / sum;
    const int64_t n_store = a.leave_tail ? nv : a.row_len;
    for (int64_t i = threadIdx.x; i < n_store; i += blockDim.x) {
        float o = 0.0f;
        if (i < nv) o = (F32_OUT ? ActVec<OT>::load1(out, i) : expf((in[i] - m) * a.scale)) * inv;
        ActVec<OT>::store1(out, i, o);
    }
}

}  // namespace

namespace {
// Persistent ring form; false = not applicable or switched off.
template <typename OT>
bool softmax_try_ring(agn_ctx *ctx, const SoftmaxArgs &a) {
    if (ctx->tune_softmax_ring == 0 || a.in == static_cast<const float *>(a.out)) return false;  // (in place: a later row's copy could overtake an earlier row's stores only if rows overlapped; rows do not, but keep the simple rule)
    const int64_t n4 = a.row_len / 4;
    int threads = (int)((n4 + 7) / 8);
    threads = ((threads + 31) / 32) * 32;
    if (threads > 1024) return false;
    const int slot_bytes = (int)((a.row_len * 4 + 127) & ~(int64_t)127);
    int slots = ctx->tune_softmax_ring >= 2 ? ctx->tune_softmax_ring : 3;
    while (slots > 2 && (size_t)slots * slot_bytes > 96 * 1024) slots--;
    const size_t smem = (size_t)slots * slot_bytes + 8 * (size_t)slots;
    if (smem > 200 * 1024) return false;
    auto kernel = softmax_ring_kernel<OT, 8>;
    int per_sm = agn_ring_ctas_per_sm(ctx, kernel, threads, smem);
    if (per_sm < 1) return false;
    if (ctx->tune_softmax_ring_ctas > 0 && ctx->tune_softmax_ring_ctas < per_sm) per_sm = ctx->tune_softmax_ring_ctas;
    int64_t grid = (int64_t)per_sm * ctx->sm_count;
    if (a.n_rows < 2 * grid && !ctx->tune_ring_force) return false;
    if (grid > a.n_rows) grid = a.n_rows;
    agn_launch(ctx, kernel, dim3((unsigned)grid), dim3(threads), smem, a, slots, slot_bytes, ctx->mbar_spin_limit, ctx->d_flags);
    ctx->flags_dirty = true;
    return true;
}

template <typename OT>
int32_t softmax_dispatch(agn_ctx *ctx, const float *in, OT *out, float *sums, int64_t n_rows, int64_t row_len,
                         int64_t row_stride, const int32_t *n_valid, int32_t causal_period, int32_t causal_offset,
                         float scale = 1.0f, bool leave_tail = false) {
    if (!(scale > 0.0f) || !(scale < INFINITY))
        return agn_fail(ctx, AGN_EINVAL, "softmax_rows: scale %g is not a positive finite number", (double)scale);
    if (n_rows < 0 || row_len < 0 || row_stride < row_len || causal_period < 0 || causal_offset < 0)
        return agn_fail(ctx, AGN_EINVAL, "softmax_rows: n_rows=%lld row_len=%lld row_stride=%lld period=%d offset=%d",
                        (long long)n_rows, (long long)row_len, (long long)row_stride, causal_period, causal_offset);
    if (n_rows == 0 || row_len == 0) return AGN_OK;
    if (!in || !out) return agn_fail(ctx, AGN_EINVAL, "softmax_rows: null pointer");
    if (n_rows > 0x7fffffffLL) return agn_fail(ctx, AGN_EINVAL, "softmax_rows: n_rows too large");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    SoftmaxArgs a;
    a.in = in; a.out = out; a.sums = sums; a.n_valid = n_valid; a.n_rows = n_rows; a.row_len = row_len; a.row_stride = row_stride;
    a.causal_period = causal_period; a.causal_offset = causal_offset;
    a.scale = scale;
    a.leave_tail = leave_tail ? 1 : 0;
    a.exp_coef = scale == 1.0f ? 1.4426950408889634f : (float)((double)scale * 1.4426950408889634);
    const bool vec_ok = row_len % 4 == 0 && row_stride % 4 == 0 && agn_aligned16(in) && agn_aligned(out, ActVec<OT>::ALIGN);
    const int64_t n4 = row_len / 4;
    if (vec_ok && n4 <= 8) {
        const unsigned grid = (unsigned)((n_rows + 255) / 256);
        if (n4 <= 2) agn_launch(ctx, softmax_thread_rows_kernel<OT, 2>, dim3(grid), dim3(256), 0, a);
        else if (n4 <= 4) agn_launch(ctx, softmax_thread_rows_kernel<OT, 4>, dim3(grid), dim3(256), 0, a);
        else agn_launch(ctx, softmax_thread_rows_kernel<OT, 8>, dim3(grid), dim3(256), 0, a);
        AGN_LAUNCHED(ctx, "softmax_thread_rows");
    } else if (vec_ok && (n4 <= 256 || (n4 <= 512 && ctx->tune_softmax_warp16))) {
        // one warp per row, statistics by shuffles alone; rows of 1025-2048 entries (sixteen float4 per
        // lane) too: a prefill's causal rows are this long, half of them mostly masked, and a CTA per
        // row with its two block-wide barriers is then bound by CTA turnover, not by HBM
        const int warps = 8;
        const unsigned grid = (unsigned)((n_rows + warps - 1) / warps);
        if (n4 <= 32) agn_launch(ctx, softmax_warp_rows_kernel<OT, 1>, dim3(grid), dim3(32 * warps), 0, a);
        else if (n4 <= 64) agn_launch(ctx, softmax_warp_rows_kernel<OT, 2>, dim3(grid), dim3(32 * warps), 0, a);
        else if (n4 <= 128) agn_launch(ctx, softmax_warp_rows_kernel<OT, 4>, dim3(grid), dim3(32 * warps), 0, a);
        else if (n4 <= 256) agn_launch(ctx, softmax_warp_rows_kernel<OT, 8>, dim3(grid), dim3(32 * warps), 0, a);
        else agn_launch(ctx, softmax_warp_rows_kernel<OT, 16>, dim3(grid), dim3(32 * warps), 0, a);
        AGN_LAUNCHED(ctx, "softmax_warp_rows");
    } else if (vec_ok && n4 > 4096 && ctx->tune_softmax_cluster && n_rows <= 0x7fffffffLL / 8 && n4 <= 8 * 16 * 512) {
        // 2..8 CTAs (the portable cluster limit) of <= 512 threads; 8 float4 per thread, or 16 for rows
        // of more than 131072 entries (a sampler's softmax over a 150K-entry vocabulary: few rows, so
        // the registers of the wider variant cost no occupancy that matters)
        const int tmax = ctx->tune_softmax_cluster == 2 && n4 <= 8 * 8 * 256 ? 256 : 512;  // measured: fewer, larger CTAs are faster
        const int vpt = n4 > 8 * 8 * 512 ? 16 : 8;
        const int cs = (int)((n4 + vpt * tmax - 1) / (vpt * tmax));
        const int threads = (int)(((n4 + vpt * cs - 1) / (vpt * cs) + 31) / 32 * 32);  // an even share, no idle tile
        if (vpt == 8)
            agn_launch_cluster(ctx, softmax_cluster_rows_kernel<OT, 8>, dim3((unsigned)(n_rows * cs)), dim3(threads), 0, cs, a, cs);
        else
            agn_launch_cluster(ctx, softmax_cluster_rows_kernel<OT, 16>, dim3((unsigned)(n_rows * cs)), dim3(threads), 0, cs, a, cs);
        AGN_LAUNCHED(ctx, "softmax_cluster_rows");
    } else if (vec_ok && n4 <= 8192 && softmax_try_ring<OT>(ctx, a)) {
        AGN_LAUNCHED(ctx, "softmax_ring");
    } else if (vec_ok && n4 <= 8192 && ctx->tune_softmax_causal_pair && !n_valid && causal_period == row_len && causal_offset == 0 &&
               n_rows % row_len == 0) {
        // square causal matrices: rows i and L-1-i share a CTA, L + 1 valid entries per CTA (nine
        // float4 per thread: eight and the one or two vectors by which the two rounded-up halves exceed a row)
        // (four float4 and a spare per thread with twice the threads measured 124 against 86 us on 28 x 2048^2)
        int threads = (int)((n4 + 7) / 8);
        threads = ((threads + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        const int64_t heads = n_rows / row_len;
        const int64_t grid = heads * ((row_len + 1) / 2);
        agn_launch(ctx, softmax_causal_pair_kernel<OT, 9>, dim3((unsigned)grid), dim3(threads), 0, a);
        AGN_LAUNCHED(ctx, "softmax_causal_pair");
    } else if (vec_ok && n4 <= 8192) {
        // few, fat threads: 8 float4 per thread keeps the CTA at <= 256 threads up to 8192 entries
        // (fewer warps in the two block-wide reductions, more loads in flight per thread)
        int vpt = 8;
        int threads = (int)((n4 + vpt - 1) / vpt);
        threads = ((threads + 31) / 32) * 32;
        if (ctx->tune_softmax_vpt == 2 || ctx->tune_softmax_vpt == 4) {
            vpt = ctx->tune_softmax_vpt;
            threads = (int)((n4 + vpt - 1) / vpt);
            threads = ((threads + 31) / 32) * 32;
            while (threads > 1024) { vpt *= 2; threads = (int)(((n4 + vpt - 1) / vpt + 31) / 32 * 32); }
        }
        if (vpt == 2) agn_launch(ctx, softmax_block_rows_kernel<OT, 2>, dim3((unsigned)n_rows), dim3(threads), 0, a);
        else if (vpt == 4) agn_launch(ctx, softmax_block_rows_kernel<OT, 4>, dim3((unsigned)n_rows), dim3(threads), 0, a);
        else agn_launch(ctx, softmax_block_rows_kernel<OT, 8>, dim3((unsigned)n_rows), dim3(threads), 0, a);
        AGN_LAUNCHED(ctx, "softmax_block_rows");
    } else {
        agn_launch(ctx, softmax_generic_rows_kernel<OT>, dim3((unsigned)n_rows), dim3(256), 0, a);
        AGN_LAUNCHED(ctx, "softmax_generic_rows");
    }
    return AGN_OK;
}
}  // namespace

extern "C" int32_t agn_softmax_rows_f32(agn_ctx *ctx, const float *in, float *out, int64_t n_rows, int64_t row_len,
                                        int64_t row_stride, const int32_t *n_valid, int32_t causal_period,
                                        int32_t causal_offset) {
    AGN_CHECK_CTX(ctx);
    return softmax_dispatch<float>(ctx, in, out, nullptr, n_rows, row_len, row_stride, n_valid, causal_period, causal_offset);
}

// The softmax step of the reference's GPU attention exactly as its kernel leaves it
// (`attention_softmax`, src/ops/kernels_wgpu.rs:795-864): weights = exp(s - max) without the
// division, sums[row] = their sum; the division is left to the consumer (`attention_output`
// divides by sums[h], :866-898).
extern "C" int32_t agn_softmax_rows_unnorm_f32(agn_ctx *ctx, const float *in, float *weights, float *sums, int64_t n_rows,
                                               int64_t row_len, int64_t row_stride, const int32_t *n_valid,
                                               int32_t causal_period, int32_t causal_offset) {
    AGN_CHECK_CTX(ctx);
    if (n_rows > 0 && !sums) return agn_fail(ctx, AGN_EINVAL, "softmax_rows_unnorm: null sums");
    return softmax_dispatch<float>(ctx, in, weights, sums, n_rows, row_len, row_stride, n_valid, causal_period, causal_offset);
}

// Softmax of scale * scores: the reference's GPU attention writes `dot * scale` with
// scale = 1 / sqrt(head_dim) in a kernel of its own (`attention_scores`,
// src/ops/kernels_wgpu.rs:773-782; the CPU path divides by sqrt(head_dim),
// src/model/llama/cpu_path.rs:172) and then runs the softmax over that buffer.  Taking the
// scale here lets the caller hand over raw dot products and saves that pass.  scale must be
// positive and finite.  sums == NULL: normalised probabilities; else exp(scale * (s - max))
// and the row sums, as agn_softmax_rows_unnorm_f32.
extern "C" int32_t agn_softmax_rows_scaled_f32(agn_ctx *ctx, const float *in, float *out, float *sums, int64_t n_rows,
                                               int64_t row_len, int64_t row_stride, const int32_t *n_valid,
                                               int32_t causal_period, int32_t causal_offset, float scale) {
    AGN_CHECK_CTX(ctx);
    return softmax_dispatch<float>(ctx, in, out, sums, n_rows, row_len, row_stride, n_valid, causal_period, causal_offset, scale);
}

// The same with the probabilities stored as f16 (out_dtype = AGN_F16) or bf16 (AGN_BF16), round to
// nearest even of the f32 value: the operand of a half-precision weights x V product, and two
// thirds of a causal softmax's traffic is the output row.  The scores stay f32; sums (optional,
// f32) as in agn_softmax_rows_scaled_f32.  out must not alias in.  No counterpart in the
// reference, whose attention weights are f32 (src/ops/kernels_wgpu.rs:795-864).
extern "C" int32_t agn_softmax_rows_scaled_f32_out16(agn_ctx *ctx, const float *in, void *out, float *sums, int64_t n_rows,
                                                     int64_t row_len, int64_t row_stride, const int32_t *n_valid,
                                                     int32_t causal_period, int32_t causal_offset, float scale,
                                                     int32_t out_dtype) {
    AGN_CHECK_CTX(ctx);
    if (out == static_cast<const void *>(in) && n_rows > 0)
        return agn_fail(ctx, AGN_EINVAL, "softmax_rows_scaled_f32_out16: a 16-bit output row cannot alias the f32 scores");
    if (out_dtype == AGN_F16)
        return softmax_dispatch<__half>(ctx, in, static_cast<__half *>(out), sums, n_rows, row_len, row_stride, n_valid,
                                        causal_period, causal_offset, scale);
    if (out_dtype == AGN_BF16)
        return softmax_dispatch<__nv_bfloat16>(ctx, in, static_cast<__nv_bfloat16 *>(out), sums, n_rows, row_len, row_stride,
                                               n_valid, causal_period, causal_offset, scale);
    return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "softmax_rows_scaled_f32_out16: output type %d is neither f16 nor bf16", out_dtype);
}

// The reference's CPU loop runs over `scores[..seq_len]` only (src/model/llama/cpu_path.rs:168-183):
// this form leaves the output entries past a row's valid length untouched instead of writing 0.
extern "C" int32_t agn_softmax_rows_valid_f32(agn_ctx *ctx, const float *in, void *out, float *sums, int64_t n_rows,
                                              int64_t row_len, int64_t row_stride, const int32_t *n_valid,
                                              int32_t causal_period, int32_t causal_offset, float scale, int32_t out_dtype) {
    AGN_CHECK_CTX(ctx);
    if (out_dtype == AGN_F32)
        return softmax_dispatch<float>(ctx, in, static_cast<float *>(out), sums, n_rows, row_len, row_stride, n_valid, causal_period,
                                       causal_offset, scale, true);
    if (out == static_cast<const void *>(in) && n_rows > 0)
        return agn_fail(ctx, AGN_EINVAL, "softmax_rows_valid_f32: a 16-bit output row cannot alias the f32 scores");
    if (out_dtype == AGN_F16)
        return softmax_dispatch<__half>(ctx, in, static_cast<__half *>(out), sums, n_rows, row_len, row_stride, n_valid,
                                        causal_period, causal_offset, scale, true);
    if (out_dtype == AGN_BF16)
        return softmax_dispatch<__nv_bfloat16>(ctx, in, static_cast<__nv_bfloat16 *>(out), sums, n_rows, row_len, row_stride,
                                               n_valid, causal_period, causal_offset, scale, true);
    return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "softmax_rows_valid_f32: output type %d is not f32, f16 or bf16", out_dtype);
}
