// Dequant-fused operand staging for the tcgen05 GEMM ("MMQ"): producer warps read packed
// weight blocks (Q4_K / Q6_K / Q8_0 / Q4_0 / NVFP4, or block-scaled fp8), decode 64 values of one
// weight row to bf16 in registers with the scales folded in, and hand them on eight values at a time:
// the GEMM's producers write them into tensor memory (the MMA's A operand), the row decoder writes
// them to a bf16 matrix.
//
// Folding the scales during staging (not in the epilogue) is the lesson of the reference's first
// tensor-core MMQ revision, whose fp32 scale epilogue took ~75 % of kernel time
// (oxidize-c/src/backends/cuda_mmq.cu:1885-1892); its kernels are k_mmq_gemm_xh_q4k / _q6k
// (:2158) on mma.sync.m16n8k8.
#pragma once
#include <cuda_fp8.h>
#include "common.cuh"
#include "quant_blocks.cuh"

namespace oxb {

constexpr int QT_FP8B = 9;  // e4m3 codes [N, K] + f32 scale per 128 input channels

struct QwArgs {
  const uint8_t* w;      // packed rows
  size_t row_bytes;      // bytes per weight row
  const float* scales;   // FP8B only: [N, K/128]
  int scale_ld;          // FP8B only: scales per row
  int staged;            // Q4_K / Q6_K: tmW is a byte map of the packed rows (shared-memory staging is possible)
};

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

// Decode values [k0, k0+64) of the row at `rowp` into 32 packed bf16 pairs.
template <int QT>
__device__ __forceinline__ void dequant64(const uint8_t* rowp, int k0, const QwArgs& qw, int n, uint32_t* out) {
  if constexpr (QT == QT_Q4_K) {
    const uint8_t* b = rowp + (size_t)(k0 >> 8) * 144;
    const int c = (k0 & 255) >> 6;
    const uint32_t dd = *reinterpret_cast<const uint32_t*>(b);
    const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
    int sc0, m0, sc1, m1;
    scale_min_k4(2 * c, b + 4, sc0, m0);
    scale_min_k4(2 * c + 1, b + 4, sc1, m1);
    const float s0 = d * (float)sc0, o0 = dmin * (float)m0, s1 = d * (float)sc1, o1 = dmin * (float)m1;
    const uint4 qa = *reinterpret_cast<const uint4*>(b + 16 + 32 * c);
    const uint4 qb = *reinterpret_cast<const uint4*>(b + 32 + 32 * c);
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    // Two values per instruction in bf16x2: a nibble OR-ed into the mantissa of 128.0 (0x4300) is the
    // bf16 number 128 + q exactly; subtracting 128 is exact; one fused multiply-add applies scale and
    // offset (computed in fp32 inside the FMA, rounded once).  Scale and offset enter as bf16, a relative
    // 2^-9 on top of the 4-bit quantisation.  ~1.5 instructions per weight instead of ~3.5.
    const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
    const __nv_bfloat162 s0b = __floats2bfloat162_rn(s0, s0), s1b = __floats2bfloat162_rn(s1, s1);
    const __nv_bfloat162 n0b = __floats2bfloat162_rn(-o0, -o0), n1b = __floats2bfloat162_rn(-o1, -o1);
    auto dq = [&](uint32_t bits, const __nv_bfloat162 sc, const __nv_bfloat162 off) {
      __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&bits);
      v = __hfma2(__hsub2(v, k128), sc, off);
      return *reinterpret_cast<uint32_t*>(&v);
    };
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t lo = q[w] & 0x0F0F0F0Fu, hi = (q[w] >> 4) & 0x0F0F0F0Fu;
      out[w * 2] = dq(__byte_perm(lo, 0x43434343u, 0x4140), s0b, n0b);       // bytes 0, 1 (low nibbles)
      out[w * 2 + 1] = dq(__byte_perm(lo, 0x43434343u, 0x4342), s0b, n0b);   // bytes 2, 3
      out[16 + w * 2] = dq(__byte_perm(hi, 0x43434343u, 0x4140), s1b, n1b);  // high nibbles: second sub-block
      out[16 + w * 2 + 1] = dq(__byte_perm(hi, 0x43434343u, 0x4342), s1b, n1b);
    }
  } else if constexpr (QT == QT_Q6_K) {
    const uint8_t* b = rowp + (size_t)(k0 >> 8) * 210;
    const int c = (k0 & 255) >> 6, half = c >> 1, hi_nib = c & 1;
    const uint8_t* ql = b + half * 64;
    const uint8_t* qh = b + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + half * 8 + 4 * hi_nib;
    const float d = __half2float(__ushort_as_half((unsigned short)ld_u16(b + 208)));
    // quarter kq = 2*hi_nib + s (s = 0: ql[0..31], s = 1: ql[32..63]); value index = s*32 + l
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int kq = 2 * hi_nib + s;
#pragma unroll
      for (int l = 0; l < 32; l += 2) {
        const uint32_t lo2 = ld_u16(ql + s * 32 + l), h2 = ld_u16(qh + l);
        float v[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t lb = (lo2 >> (8 * e)) & 0xFF, hb = (h2 >> (8 * e)) & 0xFF;
          const int q4 = hi_nib ? (lb >> 4) : (lb & 0xF);
          const int q = (q4 | (((hb >> (2 * kq)) & 3) << 4)) - 32;
          v[e] = d * (float)sc[2 * s + ((l + e) >> 4)] * (float)q;
        }
        out[(s * 32 + l) >> 1] = pack_bf16x2(v[0], v[1]);
      }
    }
  } else if constexpr (QT == QT_Q8_0) {
    // two 34-byte blocks = 68 bytes = 17 aligned words (k0 is a multiple of 64, rows are 4-byte aligned):
    // word 0 = {d0, q0 q1}, words 1..7 = q2..q29, word 8 = {q30 q31, d1}, words 9..16 = block 1's codes
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(rowp + (size_t)(k0 >> 6) * 68);
    uint32_t x[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) x[i] = wp[i];
    const float d0 = __half2float(__ushort_as_half((unsigned short)(x[0] & 0xFFFF)));
    const float d1 = __half2float(__ushort_as_half((unsigned short)(x[8] >> 16)));
    auto pair = [](uint32_t h16, float d) {
      return pack_bf16x2(d * (float)(int8_t)(h16 & 0xFF), d * (float)(int8_t)((h16 >> 8) & 0xFF));
    };
    out[0] = pair(x[0] >> 16, d0);
#pragma unroll
    for (int i = 1; i <= 7; ++i) {
      out[2 * i - 1] = pair(x[i] & 0xFFFF, d0);
      out[2 * i] = pair(x[i] >> 16, d0);
    }
    out[15] = pair(x[8] & 0xFFFF, d0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out[16 + 2 * i] = pair(x[9 + i] & 0xFFFF, d1);
      out[16 + 2 * i + 1] = pair(x[9 + i] >> 16, d1);
    }
  } else if constexpr (QT == QT_Q4_0) {
    // two 18-byte blocks = 36 bytes = 9 aligned words: word 0 = {d0, b0 b1}, words 1..3 = b2..b13,
    // word 4 = {b14 b15, d1}, words 5..8 = block 1's bytes; byte j holds value j (low nibble) and j+16 (high)
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(rowp + (size_t)(k0 >> 6) * 36);
    uint32_t x[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) x[i] = wp[i];
    const float d0 = __half2float(__ushort_as_half((unsigned short)(x[0] & 0xFFFF)));
    const float d1 = __half2float(__ushort_as_half((unsigned short)(x[4] >> 16)));
    // h16 = bytes (j, j+1): low nibbles -> values j, j+1; high nibbles -> values j+16, j+17
    auto lo = [](uint32_t h16, float d) {
      return pack_bf16x2(d * (float)((int)(h16 & 0xF) - 8), d * (float)((int)((h16 >> 8) & 0xF) - 8));
    };
    auto hi = [](uint32_t h16, float d) {
      return pack_bf16x2(d * (float)((int)((h16 >> 4) & 0xF) - 8), d * (float)((int)((h16 >> 12) & 0xF) - 8));
    };
    uint32_t h0[8], h1[8];  // the 8 byte pairs of each block
    h0[0] = x[0] >> 16;
#pragma unroll
    for (int i = 1; i <= 3; ++i) {
      h0[2 * i - 1] = x[i] & 0xFFFF;
      h0[2 * i] = x[i] >> 16;
    }
    h0[7] = x[4] & 0xFFFF;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      h1[2 * i] = x[5 + i] & 0xFFFF;
      h1[2 * i + 1] = x[5 + i] >> 16;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      out[j] = lo(h0[j], d0);
      out[8 + j] = hi(h0[j], d0);
      out[16 + j] = lo(h1[j], d1);
      out[24 + j] = hi(h1[j], d1);
    }
  } else if constexpr (QT == QT_NVFP4) {
    const uint32_t* b = reinterpret_cast<const uint32_t*>(rowp + (size_t)(k0 >> 6) * 36);
    const uint32_t sw = b[0];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const float sc = ue4m3_half((uint8_t)(sw >> (8 * s)));
      const uint32_t w0 = b[1 + 2 * s], w1 = b[2 + 2 * s];
      // byte j (0..7) holds value j (low) and j+8 (high) of the 16-value sub-block
      float v[16];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t byte = ((j < 4 ? w0 : w1) >> (8 * (j & 3))) & 0xFF;
        v[j] = sc * e2m1_doubled((int)(byte & 0xF));
        v[j + 8] = sc * e2m1_doubled((int)(byte >> 4));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) out[s * 8 + j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    }
  } else if constexpr (QT == QT_FP8B) {
    const uint8_t* b = rowp + k0;
    const float sc = qw.scales[(size_t)n * qw.scale_ld + (k0 >> 7)];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 q = *reinterpret_cast<const uint4*>(b + 16 * c);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[i] >> (16 * h)) & 0xFFFF), __NV_E4M3);
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
          out[c * 8 + i * 2 + h] = pack_bf16x2(f.x * sc, f.y * sc);
        }
      }
    }
  }
}

// 32-bit words at a 2-byte-aligned shared-memory address: N + 1 aligned words, funnel-shifted into place
template <int N>
__device__ __forceinline__ void ld_words_align2(const uint8_t* p, uint32_t* out) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(reinterpret_cast<uintptr_t>(p) & ~uintptr_t(3));
  const uint32_t sh = (uint32_t)(reinterpret_cast<uintptr_t>(p) & 2) * 8;
  uint32_t a[N + 1];
#pragma unroll
  for (int i = 0; i < N; ++i) a[i] = w[i];
  a[N] = sh ? w[N] : 0u;  // an aligned address needs no word past the last one (and must not touch it: end of a buffer)
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = __funnelshift_r(a[i], a[i + 1], sh);
}

__device__ __forceinline__ uint32_t bf16x2_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 bits_bf16x2(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }

// Decode values [k0, k0+64) of the row at `rowp` (shared memory; Q6_K / Q8_0 / Q4_0 rows may start at any even
// byte) and hand them on eight values (four packed words) at a time: put(c, w0, w1, w2, w3) receives values
// 8c .. 8c+7.  Nothing but the chunk in hand lives in registers, so many producer warps fit on an SM.  The integer codes become bf16 through the mantissa of a
// power of two (0x4300 | q is the bf16 number 128 + q for q < 128): no integer-to-float conversions.
template <int QT, class Put>
__device__ __forceinline__ void dequant64_chunks(const uint8_t* rowp, int k0, const QwArgs& qw, int n, Put&& put) {
  if constexpr (QT == QT_Q4_K) {
    const uint8_t* b = rowp + (size_t)(k0 >> 8) * 144;  // 16-byte aligned
    const int c = (k0 & 255) >> 6;
    const uint4 hdr = *reinterpret_cast<const uint4*>(b);  // d, dmin, 12 bytes of 6-bit scales and minima
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    // sub-blocks 2c and 2c + 1 (c is the same for the whole warp)
    uint32_t sc2, m2;  // two scales / minima, one per byte
    if (c < 2) {
      sc2 = (hdr.y >> (16 * c)) & 0x3F3F;
      m2 = (hdr.z >> (16 * c)) & 0x3F3F;
    } else {
      const uint32_t lo = (hdr.w >> (16 * (c - 2))) & 0xFFFF;  // low nibble: scale, high nibble: minimum
      sc2 = (lo & 0x0F0F) | (((hdr.y >> (16 * (c - 2))) & 0xC0C0) >> 2);
      m2 = ((lo >> 4) & 0x0F0F) | (((hdr.z >> (16 * (c - 2))) & 0xC0C0) >> 2);
    }
    const float s0 = d * (float)(sc2 & 0xFF), s1 = d * (float)(sc2 >> 8);
    const float o0 = dmin * (float)(m2 & 0xFF), o1 = dmin * (float)(m2 >> 8);
    const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
    const __nv_bfloat162 s0b = __floats2bfloat162_rn(s0, s0), s1b = __floats2bfloat162_rn(s1, s1);
    const __nv_bfloat162 n0b = __floats2bfloat162_rn(-o0, -o0), n1b = __floats2bfloat162_rn(-o1, -o1);
    auto dq = [&](uint32_t nib4, uint32_t sel, const __nv_bfloat162 sc, const __nv_bfloat162 off) {
      return bf16x2_bits(__hfma2(__hsub2(bits_bf16x2(__byte_perm(nib4, 0x43434343u, sel)), k128), sc, off));
    };
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // 16 bytes of codes: values 16h .. 16h+15 (low nibbles) and 32 + 16h .. (high nibbles)
      const uint4 q = *reinterpret_cast<const uint4*>(b + 16 + 32 * c + 16 * h);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t lo0 = w[2 * j] & 0x0F0F0F0Fu, lo1 = w[2 * j + 1] & 0x0F0F0F0Fu;
        const uint32_t hi0 = (w[2 * j] >> 4) & 0x0F0F0F0Fu, hi1 = (w[2 * j + 1] >> 4) & 0x0F0F0F0Fu;
        put(2 * h + j, dq(lo0, 0x4140, s0b, n0b), dq(lo0, 0x4342, s0b, n0b), dq(lo1, 0x4140, s0b, n0b),
                          dq(lo1, 0x4342, s0b, n0b));
        put(4 + 2 * h + j, dq(hi0, 0x4140, s1b, n1b), dq(hi0, 0x4342, s1b, n1b),
                          dq(hi1, 0x4140, s1b, n1b), dq(hi1, 0x4342, s1b, n1b));
      }
    }
  } else if constexpr (QT == QT_Q6_K) {
    const uint8_t* b = rowp + (size_t)(k0 >> 8) * 210;  // 2-byte aligned
    const int c = (k0 & 255) >> 6, half = c >> 1, hi_nib = c & 1;
    uint32_t qh[8], scw[1];
    ld_words_align2<8>(b + 128 + half * 32, qh);
    ld_words_align2<1>(b + 192 + half * 8 + 4 * hi_nib, scw);  // the four int8 scales of this k-block
    const float d = __half2float(__ushort_as_half((unsigned short)ld_u16(b + 208)));
    const __nv_bfloat162 k160 = __floats2bfloat162_rn(160.f, 160.f);  // 128 (mantissa trick) + 32 (code offset)
    __nv_bfloat162 scb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = d * (float)(int8_t)((scw[0] >> (8 * i)) & 0xFF);
      scb[i] = __floats2bfloat162_rn(f, f);
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {  // quarter kq = 2*hi_nib + s: 32 values
      uint32_t ql[8];
      ld_words_align2<8>(b + half * 64 + s * 32, ql);
      const int kq = 2 * hi_nib + s;
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // 8 values per chunk
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int l4 = 2 * j + e;
          const uint32_t lo4 = (ql[l4] >> (4 * hi_nib)) & 0x0F0F0F0Fu;
          const uint32_t h2 = ((qh[l4] >> (2 * kq)) & 0x03030303u) << 4;
          const uint32_t code = lo4 | h2;
          const __nv_bfloat162 sc = scb[2 * s + (l4 >> 2)];
          o[2 * e] = bf16x2_bits(__hmul2(__hsub2(bits_bf16x2(__byte_perm(code, 0x43434343u, 0x4140)), k160), sc));
          o[2 * e + 1] = bf16x2_bits(__hmul2(__hsub2(bits_bf16x2(__byte_perm(code, 0x43434343u, 0x4342)), k160), sc));
        }
        put(4 * s + j, o[0], o[1], o[2], o[3]);
      }
    }
  } else if constexpr (QT == QT_Q8_0) {
    // two 34-byte blocks (fp16 scale + 32 int8 codes), 2-byte aligned.  A code q in [-127, 127]: t = q & 0x7F is
    // q for q >= 0 and q + 128 otherwise, so q = (128 + t) - (128 or 256); both terms are exact bf16 numbers.
    const uint8_t* b = rowp + (size_t)(k0 >> 6) * 68;
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const float d = __half2float(__ushort_as_half((unsigned short)ld_u16(b + 34 * blk)));
      const __nv_bfloat162 db = __floats2bfloat162_rn(d, d);
      uint32_t q[8];
      ld_words_align2<8>(b + 34 * blk + 2, q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t x = q[2 * j + e];
          const uint32_t t = x & 0x7F7F7F7Fu, neg = x & 0x80808080u;  // neg byte 0x80 -> subtract 256 (0x4380), else 128 (0x4300)
          o[2 * e] = bf16x2_bits(__hmul2(__hsub2(bits_bf16x2(__byte_perm(t, 0x43434343u, 0x4140)),
                                                bits_bf16x2(__byte_perm(neg, 0x43434343u, 0x4140))), db));
          o[2 * e + 1] = bf16x2_bits(__hmul2(__hsub2(bits_bf16x2(__byte_perm(t, 0x43434343u, 0x4342)),
                                                    bits_bf16x2(__byte_perm(neg, 0x43434343u, 0x4342))), db));
        }
        put(4 * blk + j, o[0], o[1], o[2], o[3]);
      }
    }
  } else {
    uint32_t v[32];
    dequant64<QT>(rowp, k0, qw, n, v);
#pragma unroll
    for (int c = 0; c < 8; ++c) put(c, v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  }
}


}  // namespace oxb
