// Dequant-fused operand staging for the tcgen05 GEMM ("MMQ"): producer warps read packed
// weight blocks (Q4_K / Q6_K / Q8_0 / Q4_0 / NVFP4, or block-scaled fp8), decode 64 values of one
// weight row to bf16 in registers with the scales folded in, and store them straight into the
// 128-byte-swizzled K-major shared-memory tile that the UMMA descriptor expects — the weights are
// never materialised as bf16 in global memory.
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

// Store one row's 64 bf16 (32 packed words) into the 128B-swizzled tile: 16-byte chunk c of row r
// lives at r*128 + ((c ^ (r & 7)) << 4), the same pattern a 128B-swizzle TMA load produces.
__device__ __forceinline__ void store_row_sw128(uint8_t* tile, int r, const uint32_t* v) {
  uint8_t* rowp = tile + r * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 u = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    *reinterpret_cast<uint4*>(rowp + ((c ^ (r & 7)) << 4)) = u;
  }
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace oxb
