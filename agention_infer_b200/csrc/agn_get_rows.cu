// Embedding get_rows with inline dequantisation (Q8_0 / Q4_K / Q6_K / Q5_K / Q5_0 / Q2_K / F16 / BF16 / F32).
//
// Reference: `quant::dequant_row` + `row_view` (src/quant/mod.rs:30-47, :97-135) and the
// codecs `dequant_q8_0` (src/quant/q8_0.rs:14-51), `get_scale_min_k4` + `dequant_q4_k`
// (src/quant/q4_k.rs:26-91), `quads` + `dequant_q6_k` (src/quant/q6_k.rs:25-77), called once
// per token by the embedding loop (src/model/llama/cpu_path.rs:865-868).  The reference
// has no GPU get_rows (it dequantises on the CPU and uploads the row per token).
//
// Bit-exact contract: the codecs are integer unpacking followed by one to three f32
// operations; every one of them is spelled with __fmul_rn / __fsub_rn so nothing is
// contracted into an FMA, and f16 -> f32 is the exact widening.
//
// Data movement: one small CTA per token.  The quantised row (2-3.4 KB) is staged into
// shared memory by one bulk asynchronous copy (TMA `cp.async.bulk`, completed on an mbarrier
// with a bounded wait; 16-byte cp.async copies for the last bytes of the table or when the
// option "get_rows_tma" is 0) — Q8_0 (34 B) and Q6_K (210 B) blocks are only 2-byte aligned,
// so they cannot be read with wide loads directly — then decoded from shared memory four
// outputs per thread and written with coalesced 128-bit streaming stores.  Traffic is dominated by the f32 output (4*row_len bytes vs <= 1.06*row_len in).
#include <cuda_fp16.h>

#include "agn_common.cuh"

namespace {

__device__ __forceinline__ float f16_bits_to_f32(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t ld_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
__device__ __forceinline__ uint32_t ld_u32_2(const uint8_t *p) {  // 4 bytes from a 2-byte aligned address
    return (uint32_t)ld_u16(p) | ((uint32_t)ld_u16(p + 2) << 16);
}

// Four small unsigned integers (one per byte of x, each < 256) minus `bias` as floats without a
// conversion instruction (I2F issues at a quarter of the rate of an FADD): byte k is placed into the
// mantissa of 2^23 (0x4B000000) by one byte permute, and (2^23 + n) - (2^23 + bias) = n - bias
// exactly, because every operand and the result are integers below 2^24.
// The arithmetic of the codecs runs on Blackwell's packed f32x2 instructions (add.rn.f32x2 /
// mul.rn.f32x2: two IEEE round-to-nearest results per instruction, bit-identical to the scalar
// operations), which halves the floating-point instructions of kernels that are bound by
// instruction issue rather than by HBM.
__device__ __forceinline__ float4 bytes_minus_bias_to_float4(uint32_t x, float two23_plus_bias) {
    const float2 nb = make_float2(-two23_plus_bias, -two23_plus_bias);
    const float2 lo = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)),
                                             __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541))), nb);
    const float2 hi = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)),
                                             __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543))), nb);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
// d * q, one rounding each
__device__ __forceinline__ float4 scale4(float4 q, float d) {
    const float2 dd = make_float2(d, d);
    const float2 lo = __fmul2_rn(make_float2(q.x, q.y), dd), hi = __fmul2_rn(make_float2(q.z, q.w), dd);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Four consecutive outputs starting at element e0 (a multiple of 4) of a staged row (the
// formats whose blocks decode in element order; the K-quants have decode8 below).
template <int DTYPE>
__device__ __forceinline__ float4 decode4(const uint8_t *row, int e0);

template <>
__device__ __forceinline__ float4 decode4<AGN_Q8_0>(const uint8_t *row, int e0) {
    const uint8_t *blk = row + (e0 >> 5) * 34;
    const float d = f16_bits_to_f32(ld_u16(blk));
    const uint32_t q = ld_u32_2(blk + 2 + (e0 & 31));
    // int8 -> float: flip the sign bit (the byte becomes value + 128 in 0..255), then subtract 2^23 + 128
    return scale4(bytes_minus_bias_to_float4(q ^ 0x80808080u, 8388736.0f), d);
}

template <>
__device__ __forceinline__ float4 decode4<AGN_Q5_0>(const uint8_t *row, int e0) {
    // src/quant/q5_0.rs:20-62: f16 d, 32 high bits, 16 bytes of nibbles; value = (q - 16) * d
    const uint8_t *blk = row + (e0 >> 5) * 22;
    const int i0 = e0 & 31;
    const int hi = i0 >> 4;  // outputs 16..31 take the high nibbles and qh bits 16..31
    const int j = i0 & 15;
    const float d = f16_bits_to_f32(ld_u16(blk));
    const uint32_t qh = ld_u32_2(blk + 2) >> (j + 16 * hi);
    const uint32_t q = ld_u32_2(blk + 6 + j) >> (4 * hi);
    float4 o;
    o.x = __fmul_rn((float)((int)((q & 0xF) | ((qh & 1) << 4)) - 16), d);
    o.y = __fmul_rn((float)((int)(((q >> 8) & 0xF) | (((qh >> 1) & 1) << 4)) - 16), d);
    o.z = __fmul_rn((float)((int)(((q >> 16) & 0xF) | (((qh >> 2) & 1) << 4)) - 16), d);
    o.w = __fmul_rn((float)((int)(((q >> 24) & 0xF) | (((qh >> 3) & 1) << 4)) - 16), d);
    return o;
}

template <>
__device__ __forceinline__ float4 decode4<AGN_F16>(const uint8_t *row, int e0) {
    const uint8_t *p = row + 2 * e0;
    return make_float4(f16_bits_to_f32(ld_u16(p)), f16_bits_to_f32(ld_u16(p + 2)), f16_bits_to_f32(ld_u16(p + 4)),
                       f16_bits_to_f32(ld_u16(p + 6)));
}

template <>
__device__ __forceinline__ float4 decode4<AGN_BF16>(const uint8_t *row, int e0) {
    const uint8_t *p = row + 2 * e0;
    return make_float4(__uint_as_float((uint32_t)ld_u16(p) << 16), __uint_as_float((uint32_t)ld_u16(p + 2) << 16),
                       __uint_as_float((uint32_t)ld_u16(p + 4) << 16), __uint_as_float((uint32_t)ld_u16(p + 6) << 16));
}

template <>
__device__ __forceinline__ float4 decode4<AGN_F32>(const uint8_t *row, int e0) {
    const uint8_t *p = row + 4 * e0;
    return make_float4(__uint_as_float(ld_u32_2(p)), __uint_as_float(ld_u32_2(p + 4)), __uint_as_float(ld_u32_2(p + 8)),
                       __uint_as_float(ld_u32_2(p + 12)));
}

// Eight outputs per call: two float4 at elements ea and eb of the row.  For the K-quants the
// two float4 are the low- and the high-nibble values of the same four quant bytes, so the
// bytes, the super-block scales and (Q5_K, Q6_K) the high-bit word are loaded and unpacked
// once for both; eight consecutive units still write 128 contiguous bytes per float4.
template <int DTYPE>
__device__ __forceinline__ void decode8(const uint8_t *row, int u, int row_len, int &ea, float4 &va, int &eb, float4 &vb) {
    ea = 8 * u;
    eb = 8 * u + 4;
    va = decode4<DTYPE>(row, ea);
    vb = eb < row_len ? decode4<DTYPE>(row, eb) : make_float4(0.f, 0.f, 0.f, 0.f);
}

__device__ __forceinline__ void k4_scale_min(const uint8_t *sc, int j, uint32_t &s, uint32_t &m) {
    if (j < 4) {
        s = sc[j] & 63;
        m = sc[j + 4] & 63;
    } else {
        s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4);
        m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
    }
}

template <>
__device__ __forceinline__ void decode8<AGN_Q4_K>(const uint8_t *row, int u, int, int &ea, float4 &va, int &eb, float4 &vb) {
    const uint8_t *blk = row + (u >> 5) * 144;
    const int r = u & 31, g = r >> 3, l = (r & 7) * 4;
    ea = (u >> 5) * 256 + 64 * g + l;
    eb = ea + 32;
    const uint32_t dm = *reinterpret_cast<const uint32_t *>(blk);
    const float d = f16_bits_to_f32((uint16_t)(dm & 0xffff));
    const float dmin = f16_bits_to_f32((uint16_t)(dm >> 16));
    uint32_t s0, m0, s1, m1;
    k4_scale_min(blk + 4, 2 * g, s0, m0);
    k4_scale_min(blk + 4, 2 * g + 1, s1, m1);
    const float d1 = __fmul_rn(d, (float)s0), mm1 = __fmul_rn(dmin, (float)m0);
    const float d2 = __fmul_rn(d, (float)s1), mm2 = __fmul_rn(dmin, (float)m1);
    const uint32_t q = *reinterpret_cast<const uint32_t *>(blk + 16 + 32 * g + l);
    va.x = __fsub_rn(__fmul_rn(d1, (float)(q & 0xF)), mm1);
    va.y = __fsub_rn(__fmul_rn(d1, (float)((q >> 8) & 0xF)), mm1);
    va.z = __fsub_rn(__fmul_rn(d1, (float)((q >> 16) & 0xF)), mm1);
    va.w = __fsub_rn(__fmul_rn(d1, (float)((q >> 24) & 0xF)), mm1);
    vb.x = __fsub_rn(__fmul_rn(d2, (float)((q >> 4) & 0xF)), mm2);
    vb.y = __fsub_rn(__fmul_rn(d2, (float)((q >> 12) & 0xF)), mm2);
    vb.z = __fsub_rn(__fmul_rn(d2, (float)((q >> 20) & 0xF)), mm2);
    vb.w = __fsub_rn(__fmul_rn(d2, (float)(q >> 28)), mm2);
}

__device__ __forceinline__ float4 bytes_to_float4(uint32_t x) { return bytes_minus_bias_to_float4(x, 8388608.0f); }
__device__ __forceinline__ float4 scale_sub4(float4 q, float d, float m) {  // d * q - m, two roundings each (x - m is x + (-m))
    const float2 dd = make_float2(d, d), nm = make_float2(-m, -m);
    const float2 lo = __fadd2_rn(__fmul2_rn(make_float2(q.x, q.y), dd), nm);
    const float2 hi = __fadd2_rn(__fmul2_rn(make_float2(q.z, q.w), dd), nm);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Q4_K, sixteen outputs per call: two 4-byte words of one 64-value group, 16 bytes apart, give
// low-nibble values at elements e and e + 16 and high-nibble values at e + 32 and e + 48 (four
// neighbouring lanes then write 64 contiguous bytes with every store instruction).  The block header (d, dmin and the
// twelve packed scale bytes, src/quant/q4_k.rs:26-35) is one 128-bit shared-memory load and the
// 6-bit scales are cut out of its words, shared by all sixteen outputs.  Q4_K rows are multiples
// of 144 bytes, so every block starts on a 16-byte boundary of the staging buffer.
__device__ __forceinline__ void decode16_q4_k(const uint8_t *row, int u, int &e, float4 lo[2], float4 hi[2]) {
    const uint8_t *blk = row + (u >> 4) * 144;
    const int r = u & 15, g = r >> 2, l = (r & 3) * 4;
    e = (u >> 4) * 256 + 64 * g + l;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xffff));
    const float dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
    uint32_t s0, m0, s1, m1;
    if (g < 2) {  // sub-blocks 0..3: the low six bits of scale bytes j and j + 4
        const int sh = 16 * g;
        s0 = (hdr.y >> sh) & 63;
        m0 = (hdr.z >> sh) & 63;
        s1 = (hdr.y >> (sh + 8)) & 63;
        m1 = (hdr.z >> (sh + 8)) & 63;
    } else {  // sub-blocks 4..7: a nibble of byte j + 4 and the top two bits of bytes j - 4 and j
        const int sh = 16 * (g - 2);
        s0 = ((hdr.w >> sh) & 0xF) | (((hdr.y >> (sh + 6)) & 3) << 4);
        m0 = ((hdr.w >> (sh + 4)) & 0xF) | (((hdr.z >> (sh + 6)) & 3) << 4);
        s1 = ((hdr.w >> (sh + 8)) & 0xF) | (((hdr.y >> (sh + 14)) & 3) << 4);
        m1 = ((hdr.w >> (sh + 12)) & 0xF) | (((hdr.z >> (sh + 14)) & 3) << 4);
    }
    const float d1 = __fmul_rn(d, (float)s0), mm1 = __fmul_rn(dmin, (float)m0);
    const float d2 = __fmul_rn(d, (float)s1), mm2 = __fmul_rn(dmin, (float)m1);
    const uint32_t qa = *reinterpret_cast<const uint32_t *>(blk + 16 + 32 * g + l);
    const uint32_t qb = *reinterpret_cast<const uint32_t *>(blk + 32 + 32 * g + l);
    lo[0] = scale_sub4(bytes_to_float4(qa & 0x0F0F0F0Fu), d1, mm1);
    lo[1] = scale_sub4(bytes_to_float4(qb & 0x0F0F0F0Fu), d1, mm1);
    hi[0] = scale_sub4(bytes_to_float4((qa >> 4) & 0x0F0F0F0Fu), d2, mm2);
    hi[1] = scale_sub4(bytes_to_float4((qb >> 4) & 0x0F0F0F0Fu), d2, mm2);
}

template <>
__device__ __forceinline__ void decode8<AGN_Q5_K>(const uint8_t *row, int u, int, int &ea, float4 &va, int &eb, float4 &vb) {
    const uint8_t *blk = row + (u >> 5) * 176;
    const int r = u & 31, g = r >> 3, l = (r & 7) * 4;
    ea = (u >> 5) * 256 + 64 * g + l;
    eb = ea + 32;
    const uint32_t dm = *reinterpret_cast<const uint32_t *>(blk);
    const float d = f16_bits_to_f32((uint16_t)(dm & 0xffff));
    const float dmin = f16_bits_to_f32((uint16_t)(dm >> 16));
    uint32_t s0, m0, s1, m1;
    k4_scale_min(blk + 4, 2 * g, s0, m0);
    k4_scale_min(blk + 4, 2 * g + 1, s1, m1);
    const float d1 = __fmul_rn(d, (float)s0), mm1 = __fmul_rn(dmin, (float)m0);
    const float d2 = __fmul_rn(d, (float)s1), mm2 = __fmul_rn(dmin, (float)m1);
    const uint32_t qh = *reinterpret_cast<const uint32_t *>(blk + 16 + l) >> (2 * g);  // bit 0: low run, bit 1: high run
    const uint32_t q = *reinterpret_cast<const uint32_t *>(blk + 48 + 32 * g + l);
    // four 5-bit values per word, a byte each: nibble plus the high bit (bit 0 of the qh byte for the low run, bit 1 for the high run)
    va = scale_sub4(bytes_to_float4((q & 0x0F0F0F0Fu) | ((qh & 0x01010101u) << 4)), d1, mm1);
    vb = scale_sub4(bytes_to_float4(((q >> 4) & 0x0F0F0F0Fu) | (((qh >> 1) & 0x01010101u) << 4)), d2, mm2);
}

template <>
__device__ __forceinline__ void decode8<AGN_Q2_K>(const uint8_t *row, int u, int, int &ea, float4 &va, int &eb, float4 &vb) {
    // src/quant/q2_k.rs:47-93: scales[16] | qs[64] | f16 d | f16 dmin; value e of the super-block is
    // ((qs[32*(e/128) + e%32] >> 2*((e%128)/32)) & 3) * d*(scales[e/16] & 0xF) - dmin*(scales[e/16] >> 4).
    // One unit = four quant bytes at two adjacent shifts (outputs 32 apart).
    const uint8_t *blk = row + (u >> 5) * 84;
    const int r = u & 31, g = r >> 4, jp = (r >> 3) & 1, l = (r & 7) * 4;
    const int e = 128 * g + 64 * jp + l;
    ea = (u >> 5) * 256 + e;
    eb = ea + 32;
    const uint32_t dm = *reinterpret_cast<const uint32_t *>(blk + 80);
    const float d = f16_bits_to_f32((uint16_t)(dm & 0xffff));
    const float dmin = f16_bits_to_f32((uint16_t)(dm >> 16));
    const uint32_t sa = blk[e >> 4], sb = blk[(e >> 4) + 2];
    const float d1 = __fmul_rn(d, (float)(sa & 0xF)), mm1 = __fmul_rn(dmin, (float)(sa >> 4));
    const float d2 = __fmul_rn(d, (float)(sb & 0xF)), mm2 = __fmul_rn(dmin, (float)(sb >> 4));
    const uint32_t q = *reinterpret_cast<const uint32_t *>(blk + 16 + 32 * g + l) >> (4 * jp);
    va = scale_sub4(bytes_to_float4(q & 0x03030303u), d1, mm1);
    vb = scale_sub4(bytes_to_float4((q >> 2) & 0x03030303u), d2, mm2);
}

template <>
__device__ __forceinline__ void decode8<AGN_Q6_K>(const uint8_t *row, int u, int, int &ea, float4 &va, int &eb, float4 &vb) {
    const uint8_t *blk = row + (u >> 5) * 210;
    const int r = u & 31, h = r >> 4, cp = (r >> 3) & 1, l = (r & 7) * 4;
    ea = (u >> 5) * 256 + 128 * h + 32 * cp + l;  // quadrant cp: low nibbles
    eb = ea + 64;                                 // quadrant cp + 2: high nibbles of the same bytes
    const uint32_t ql = ld_u32_2(blk + h * 64 + cp * 32 + l);
    const uint32_t qh = ld_u32_2(blk + 128 + h * 32 + l) >> (2 * cp);
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * h + (l >> 4) + 2 * cp);
    const float d = f16_bits_to_f32(ld_u16(blk + 208));
    const float da = __fmul_rn(d, (float)sc[0]), db = __fmul_rn(d, (float)sc[4]);
    // four 6-bit values per word, a byte each: low (high) nibbles of ql with bits 0-1 (4-5) of the qh bytes on top;
    // value - 32 comes out of the byte-to-float step (2^23 + 32 is subtracted)
    const float4 fa = bytes_minus_bias_to_float4((ql & 0x0F0F0F0Fu) | ((qh & 0x03030303u) << 4), 8388640.0f);
    const float4 fb = bytes_minus_bias_to_float4(((ql >> 4) & 0x0F0F0F0Fu) | (((qh >> 4) & 0x03030303u) << 4), 8388640.0f);
    va = scale4(fa, da);
    vb = scale4(fb, db);
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

// --- staging of the quantised row into shared memory ---------------------------------------
// Preferred: one bulk asynchronous copy (TMA, `cp.async.bulk` into this CTA's own shared memory) issued by one
// thread and completed on an mbarrier; it needs 16-byte aligned source, destination and size,
// which holds whenever the 16-byte rounded row lies inside the table.  Otherwise (the last
// bytes of the table) 16-byte cp.async copies with a byte-wise tail.
// Decodes a staged row and writes its row_len outputs.
template <int DTYPE, typename OUT, bool VEC_OUT>
__device__ __forceinline__ void decode_row(const uint8_t *row, int row_len, OUT *o_row) {
    // a partial last block is fully present in the table (type_size rounds up to whole blocks),
    // so decoding past row_len inside it stays in bounds; only the stores are clipped
    // K-quant units are numbered per 256-value super-block (32 units each, not in element order)
    constexpr bool K_QUANT = DTYPE == AGN_Q4_K || DTYPE == AGN_Q5_K || DTYPE == AGN_Q6_K || DTYPE == AGN_Q2_K;
    if (DTYPE == AGN_Q4_K && VEC_OUT) {
        const int n16 = ((row_len + 255) >> 8) * 16;
        for (int u = threadIdx.x; u < n16; u += blockDim.x) {
            int e;
            float4 lo[2], hi[2];
            decode16_q4_k(row, u, e, lo, hi);
            if (e < row_len) ActVec<OUT>::store(o_row, e >> 2, lo[0]);
            if (e + 16 < row_len) ActVec<OUT>::store(o_row, (e >> 2) + 4, lo[1]);
            if (e + 32 < row_len) ActVec<OUT>::store(o_row, (e >> 2) + 8, hi[0]);
            if (e + 48 < row_len) ActVec<OUT>::store(o_row, (e >> 2) + 12, hi[1]);
        }
        return;
    }
    const int n8 = K_QUANT ? ((row_len + 255) >> 8) * 32 : (row_len + 7) >> 3;
    for (int u = threadIdx.x; u < n8; u += blockDim.x) {
        int ea, eb;
        float4 va, vb;
        decode8<DTYPE>(row, u, row_len, ea, va, eb, vb);
        if (VEC_OUT) {
            if (ea < row_len) ActVec<OUT>::store(o_row, ea >> 2, va);
            if (eb < row_len) ActVec<OUT>::store(o_row, eb >> 2, vb);
        } else {
            const float a[4] = {va.x, va.y, va.z, va.w}, b[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (ea + i < row_len) ActVec<OUT>::store1(o_row, ea + i, a[i]);
                if (eb + i < row_len) ActVec<OUT>::store1(o_row, eb + i, b[i]);
            }
        }
    }
}

// 16-byte cp.async copies of the 16-byte-rounded row, byte-wise for a last chunk that would
// reach past the end of the table.
__device__ __forceinline__ void stage_row_chunks(uint8_t *stage, const uint8_t *table, size_t table_bytes, size_t a0, int n16) {
    for (int c = threadIdx.x; c < n16; c += blockDim.x) {
        const size_t off = a0 + 16 * (size_t)c;
        if (off + 16 <= table_bytes) {
            cp_async16(stage + 16 * c, table + off);
        } else {
            for (int b = 0; b < 16; b++) stage[16 * c + b] = off + b < table_bytes ? table[off + b] : 0;
        }
    }
    cp_async_wait_all();
}

template <int DTYPE, typename OUT, bool VEC_OUT, bool TMA>
__global__ void __launch_bounds__(256)
get_rows_kernel(const uint8_t *__restrict__ table, size_t table_bytes, int64_t n_rows, int row_len, int row_bytes,
                const uint32_t *__restrict__ ids, OUT *__restrict__ out, uint32_t *flags, int spin_limit, int test_idle_wait) {
    extern __shared__ __align__(128) uint8_t stage[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ __align__(8) uint64_t idle_bar;  // test hook only: initialised, never signalled
    if (TMA) {
        if (threadIdx.x == 0) {
            agn_mbar_init(&bar, 1);
            agn_mbar_init(&idle_bar, 1);
            agn_mbar_init_fence();
        }
        __syncthreads();  // barrier initialised before anyone polls it (runs ahead of the dependency wait)
    }
    agn_pdl_prologue();
    const int64_t t = blockIdx.x;
    const uint32_t id = ids[t];
    OUT *o_row = out + t * (int64_t)row_len;
    if ((int64_t)id >= n_rows) {
        // "row index out of range": zero row + error flag, never a trap
        for (int j = threadIdx.x; j < row_len; j += blockDim.x) ActVec<OUT>::store1(o_row, j, 0.0f);
        if (threadIdx.x == 0) atomicOr(flags, AGN_FLAG_OOB_ID);
        return;
    }
    const size_t start = (size_t)id * (size_t)row_bytes;
    const size_t a0 = start & ~(size_t)15;
    const int lead = (int)(start - a0);
    const int n16 = (lead + row_bytes + 15) >> 4;
    const bool bulk = TMA && a0 + 16 * (size_t)n16 <= table_bytes;  // same answer in every thread of the CTA
    if (bulk) {
        if (threadIdx.x == 0) {
            agn_mbar_expect_tx(&bar, 16u * (uint32_t)n16);
            agn_bulk_g2s(stage, table + a0, 16u * (uint32_t)n16, &bar);
        }
        // (with the test hook the row itself is awaited with the default limit, so that no copy is in
        // flight when the wait that is meant to run out, on the idle barrier, gives up)
        if (!agn_mbar_wait(&bar, 0, test_idle_wait ? AGN_MBAR_SPIN_LIMIT_DEFAULT : spin_limit) ||
            (test_idle_wait && !agn_mbar_wait(&idle_bar, 0, spin_limit))) {
            // report it; the copy may still be writing shared memory: wait once more, bounded, before
            // leaving.  The output row is not written.
            if (threadIdx.x == 0) atomicOr(flags, AGN_FLAG_TIMEOUT);
            (void)agn_mbar_wait(&bar, 0, spin_limit);
            return;
        }
    } else {
        stage_row_chunks(stage, table, table_bytes, a0, n16);
        __syncthreads();
    }
    decode_row<DTYPE, OUT, VEC_OUT>(stage + lead, row_len, o_row);
}

// Persistent form: a few small CTAs per SM, each looping over tokens blockIdx.x, blockIdx.x +
// gridDim.x, ...  The quantised rows of the CTA's next `slots` tokens are already on their way
// into a ring of shared-memory slots (thread 0 reads their ids and issues one bulk copy each)
// while the current row is decoded, so the id -> row address -> row bytes latency chain of a
// token is hidden behind the decode of the tokens before it.
template <int DTYPE, typename OUT, bool VEC_OUT>
__global__ void __launch_bounds__(256)
get_rows_ring_kernel(const uint8_t *__restrict__ table, size_t table_bytes, int64_t n_rows, int row_len, int row_bytes,
                     const uint32_t *__restrict__ ids, OUT *__restrict__ out, int64_t T, int slots, int slot_bytes,
                     uint32_t *flags, int spin_limit) {
    extern __shared__ __align__(128) uint8_t ring[];
    uint64_t *full = reinterpret_cast<uint64_t *>(ring + (size_t)slots * slot_bytes);
    if (threadIdx.x == 0) {
        for (int s = 0; s < slots; s++) agn_mbar_init(&full[s], 1);
        agn_mbar_init_fence();
    }
    __syncthreads();
    agn_pdl_launch_dependents();
    agn_pdl_wait();
    const int64_t first = blockIdx.x, stride = gridDim.x;
    const int n_my = first < T ? (int)((T - first + stride - 1) / stride) : 0;
    // Whether a token's row comes by bulk copy is a function of its id alone, so the issuing
    // thread and the consuming threads reach the same answer independently.
    auto row_span = [&](uint32_t id, size_t &a0, int &lead, int &n16) -> int {  // 0: id out of range, 1: bulk copy, 2: chunked copy
        if ((int64_t)id >= n_rows) return 0;
        const size_t start = (size_t)id * (size_t)row_bytes;
        a0 = start & ~(size_t)15;
        lead = (int)(start - a0);
        n16 = (lead + row_bytes + 15) >> 4;
        return a0 + 16 * (size_t)n16 <= table_bytes ? 1 : 2;
    };
    auto issue = [&](int j) {  // thread 0 only
        size_t a0; int lead, n16;
        if (row_span(ids[first + (int64_t)j * stride], a0, lead, n16) != 1) return;
        uint64_t *bar = &full[j % slots];
        agn_mbar_expect_tx(bar, 16u * (uint32_t)n16);
        agn_bulk_g2s(ring + (size_t)(j % slots) * slot_bytes, table + a0, 16u * (uint32_t)n16, bar);
    };
    if (threadIdx.x == 0)
        for (int j = 0; j < slots && j < n_my; j++) issue(j);

    // parity of a slot's barrier flips only when a bulk copy completed on it
    uint32_t phase_bits = 0;  // bit s: parity the next wait on slot s expects
    for (int it = 0; it < n_my; it++) {
        const int slot = it % slots;
        const int64_t t = first + (int64_t)it * stride;
        OUT *o_row = out + t * (int64_t)row_len;
        uint8_t *stage = ring + (size_t)slot * slot_bytes;
        size_t a0 = 0; int lead = 0, n16 = 0;
        const int kind = row_span(ids[t], a0, lead, n16);
        int failed = 0;
        if (kind == 1) {
            failed = !agn_mbar_wait(&full[slot], (phase_bits >> slot) & 1u, spin_limit);
            phase_bits ^= 1u << slot;
        } else if (kind == 2) {
            stage_row_chunks(stage, table, table_bytes, a0, n16);
            __syncthreads();
        }
        if (kind == 0) {
            for (int j = threadIdx.x; j < row_len; j += blockDim.x) ActVec<OUT>::store1(o_row, j, 0.0f);
            if (threadIdx.x == 0) atomicOr(flags, AGN_FLAG_OOB_ID);
        } else if (!failed) {
            decode_row<DTYPE, OUT, VEC_OUT>(stage + lead, row_len, o_row);
        }
        // every thread is done with the slot; one CTA-wide answer to "did any thread's wait run
        // out", so that all threads leave together
        if (__syncthreads_or(failed)) {
            // report it and give the copies still in flight (they target this
            // CTA's shared memory) one more bounded wait each before leaving
            if (threadIdx.x == 0) {
                atomicOr(flags, AGN_FLAG_TIMEOUT);
                for (int j = it; j < n_my && j < it + slots; j++) {
                    size_t b0; int l2, m16;
                    const bool waited_already = j == it;  // its parity bit has been flipped above
                    if (row_span(ids[first + (int64_t)j * stride], b0, l2, m16) == 1)
                        (void)agn_mbar_wait(&full[j % slots], ((phase_bits >> (j % slots)) & 1u) ^ (waited_already ? 1u : 0u), spin_limit);
                }
            }
            return;
        }
        if (threadIdx.x == 0 && it + slots < n_my) issue(it + slots);
    }
}

template <int DTYPE, typename OUT, bool VEC_OUT>
bool launch_get_rows_ring(agn_ctx *ctx, int threads, const uint8_t *table, size_t table_bytes, int64_t n_rows, int row_len,
                          int row_bytes, const uint32_t *ids, int64_t T, OUT *out) {
    if (ctx->tune_get_rows_ring == 0 || !ctx->tune_get_rows_tma || ctx->test_idle_barrier_wait) return false;
    const int slot_bytes = (((row_bytes + 15) / 16 + 2) * 16 + 127) & ~127;
    int slots = ctx->tune_get_rows_ring >= 2 ? ctx->tune_get_rows_ring : 4;
    while (slots > 2 && (size_t)slots * slot_bytes > 48 * 1024) slots--;
    const size_t smem = (size_t)slots * slot_bytes + 8 * (size_t)slots;
    if (smem > 200 * 1024) return false;
    auto kernel = get_rows_ring_kernel<DTYPE, OUT, VEC_OUT>;
    int per_sm = agn_ring_ctas_per_sm(ctx, kernel, threads, smem);
    if (per_sm < 1) return false;
    if (ctx->tune_get_rows_ring_ctas > 0 && ctx->tune_get_rows_ring_ctas < per_sm) per_sm = ctx->tune_get_rows_ring_ctas;
    int64_t grid = (int64_t)per_sm * ctx->sm_count;
    if (T < 2 * grid && !ctx->tune_ring_force) return false;  // too few tokens per CTA for a ring to pay
    if (grid > T) grid = T;
    agn_launch(ctx, kernel, dim3((unsigned)grid), dim3(threads), smem, table, table_bytes, n_rows, row_len, row_bytes, ids, out, T,
               slots, slot_bytes, ctx->d_flags, ctx->mbar_spin_limit);
    ctx->ring_launched = true;
    return true;
}

template <int DTYPE, typename OUT>
cudaError_t launch_get_rows(agn_ctx *ctx, bool vec, int64_t T, int threads, size_t smem, const uint8_t *table,
                            size_t table_bytes, int64_t n_rows, int row_len, int row_bytes, const uint32_t *ids, OUT *out) {
    if (vec ? launch_get_rows_ring<DTYPE, OUT, true>(ctx, threads, table, table_bytes, n_rows, row_len, row_bytes, ids, T, out)
            : launch_get_rows_ring<DTYPE, OUT, false>(ctx, threads, table, table_bytes, n_rows, row_len, row_bytes, ids, T, out))
        return cudaSuccess;
    const unsigned grid = (unsigned)T;
    cudaError_t e = cudaSuccess;
    if (smem > 48 * 1024) {  // opt in to large dynamic shared memory for very long rows
        e = cudaFuncSetAttribute(get_rows_kernel<DTYPE, OUT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(get_rows_kernel<DTYPE, OUT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(get_rows_kernel<DTYPE, OUT, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(get_rows_kernel<DTYPE, OUT, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const bool tma = ctx->tune_get_rows_tma != 0;
    const int lim = ctx->mbar_spin_limit, extra = ctx->test_idle_barrier_wait;  // extra: the idle-barrier test hook
    if (vec && tma)
        agn_launch(ctx, get_rows_kernel<DTYPE, OUT, true, true>, dim3(grid), dim3(threads), smem, table, table_bytes, n_rows, row_len, row_bytes, ids, out, ctx->d_flags, lim, extra);
    else if (vec)
        agn_launch(ctx, get_rows_kernel<DTYPE, OUT, true, false>, dim3(grid), dim3(threads), smem, table, table_bytes, n_rows, row_len, row_bytes, ids, out, ctx->d_flags, lim, extra);
    else if (tma)
        agn_launch(ctx, get_rows_kernel<DTYPE, OUT, false, true>, dim3(grid), dim3(threads), smem, table, table_bytes, n_rows, row_len, row_bytes, ids, out, ctx->d_flags, lim, extra);
    else
        agn_launch(ctx, get_rows_kernel<DTYPE, OUT, false, false>, dim3(grid), dim3(threads), smem, table, table_bytes, n_rows, row_len, row_bytes, ids, out, ctx->d_flags, lim, extra);
    return cudaSuccess;
}

template <typename OUT>
int32_t get_rows_dispatch(agn_ctx *ctx, int32_t dtype, const void *table, size_t table_bytes, int64_t n_rows, int64_t row_len,
                          const uint32_t *ids, int64_t T, OUT *out) {
    const size_t row_bytes = agn_type_size(dtype, (size_t)(row_len > 0 ? row_len : 0));
    if (dtype != AGN_Q8_0 && dtype != AGN_Q4_K && dtype != AGN_Q6_K && dtype != AGN_Q5_K && dtype != AGN_Q5_0 && dtype != AGN_Q2_K && dtype != AGN_F16 &&
        dtype != AGN_BF16 && dtype != AGN_F32)
        return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "get_rows: dequantization not implemented for ggml type %d", dtype);
    if (T < 0 || n_rows < 0 || row_len <= 0)
        return agn_fail(ctx, AGN_EINVAL, "get_rows: T=%lld n_rows=%lld row_len=%lld", (long long)T, (long long)n_rows, (long long)row_len);
    if (dtype == AGN_Q2_K && row_len % 256 != 0)  // src/quant/q2_k.rs:31-35
        return agn_fail(ctx, AGN_EINVAL, "get_rows: Q2_K row length %lld is not a multiple of 256", (long long)row_len);
    if (T == 0) return AGN_OK;
    if (!table || !ids || !out) return agn_fail(ctx, AGN_EINVAL, "get_rows: null pointer");
    if (!agn_aligned16(table)) return agn_fail(ctx, AGN_EINVAL, "get_rows: table must be 16-byte aligned");
    if (row_bytes == 0 || (size_t)n_rows > table_bytes / row_bytes)  // division: n_rows * row_bytes may not fit 64 bits
        return agn_fail(ctx, AGN_EINVAL, "get_rows: tensor rows extend beyond the data (%lld rows of %zu bytes, have %zu)",
                        (long long)n_rows, row_bytes, table_bytes);
    if (row_bytes + 32 > 200 * 1024) return agn_fail(ctx, AGN_EINVAL, "get_rows: row of %zu bytes exceeds the staging buffer", row_bytes);
    if (T > 0x7fffffffLL || row_len > 0x3fffffffLL) return agn_fail(ctx, AGN_EINVAL, "get_rows: T or row_len too large");
    AGN_CUDA(ctx, cudaSetDevice(ctx->device));
    const bool vec = row_len % 4 == 0 && agn_aligned(out, ActVec<OUT>::ALIGN);
    const int n4 = (int)((row_len + 3) / 4);
    // small CTAs (8 float4 per thread): more rows resident per SM hides the id -> row -> decode
    // latency chain better than wide CTAs do (measured: 128 threads beat 224 by 15% at H=3584)
    int threads = ((n4 + 7) / 8 + 31) / 32 * 32;  // four 8-value units per thread
    if (threads < 64) threads = 64;
    if (threads > 256) threads = 256;
    if (ctx->tune_get_rows_threads >= 32 && ctx->tune_get_rows_threads <= 256) threads = ctx->tune_get_rows_threads & ~31;
    const size_t smem = ((row_bytes + 15) / 16 + 2) * 16;
    const uint8_t *tb = static_cast<const uint8_t *>(table);
    const int rl = (int)row_len, rb = (int)row_bytes;
    cudaError_t e;
    ctx->ring_launched = false;
    switch (dtype) {
    case AGN_Q8_0: e = launch_get_rows<AGN_Q8_0, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_Q4_K: e = launch_get_rows<AGN_Q4_K, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_Q6_K: e = launch_get_rows<AGN_Q6_K, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_Q5_K: e = launch_get_rows<AGN_Q5_K, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_Q2_K: e = launch_get_rows<AGN_Q2_K, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_Q5_0: e = launch_get_rows<AGN_Q5_0, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_F16: e = launch_get_rows<AGN_F16, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    case AGN_BF16: e = launch_get_rows<AGN_BF16, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    default: e = launch_get_rows<AGN_F32, OUT>(ctx, vec, T, threads, smem, tb, table_bytes, n_rows, rl, rb, ids, out); break;
    }
    AGN_CUDA(ctx, e);
    ctx->flags_dirty = true;
    if (ctx->ring_launched) AGN_LAUNCHED(ctx, "get_rows_ring");
    else AGN_LAUNCHED(ctx, "get_rows");
    return AGN_OK;
}

}  // namespace

extern "C" int32_t agn_get_rows_f32(agn_ctx *ctx, int32_t dtype, const void *table, size_t table_bytes, int64_t n_rows,
                                    int64_t row_len, const uint32_t *ids, int64_t T, float *out) {
    AGN_CHECK_CTX(ctx);
    return get_rows_dispatch<float>(ctx, dtype, table, table_bytes, n_rows, row_len, ids, T, out);
}

// Output stored as f16 (round to nearest even): the embedding row as the reference uploads
// it with `Act = f16` (`act_encode`, src/ops/mod.rs:47-60, after the CPU `dequant_row`).
extern "C" int32_t agn_get_rows_f16(agn_ctx *ctx, int32_t dtype, const void *table, size_t table_bytes, int64_t n_rows,
                                    int64_t row_len, const uint32_t *ids, int64_t T, void *out) {
    AGN_CHECK_CTX(ctx);
    return get_rows_dispatch<__half>(ctx, dtype, table, table_bytes, n_rows, row_len, ids, T, static_cast<__half *>(out));
}
