// Device-side decoders for the GGUF block formats (little-endian layouts as in
// oxidize-core/src/compute/quantization.rs:5-53): Q8_0 34 B/32, Q4_0 18 B/32, Q4_K 144 B/256,
// Q5_K 176 B/256, Q6_K 210 B/256, NVFP4 36 B/64.  Decode math follows the reference kernels
// dequant_q4_k / dequant_q6_k / dequant_nvfp4 (kernels/gemv_f32.cu:253,284,1513) and
// get_scale_min_k4 (:240-250).
#pragma once
#include "common.cuh"

namespace oxb {

enum QType : int {
  QT_F32 = 0,
  QT_F16 = 1,
  QT_BF16 = 2,
  QT_Q8_0 = 3,
  QT_Q4_0 = 4,
  QT_Q4_K = 5,
  QT_Q5_K = 6,
  QT_Q6_K = 7,
  QT_NVFP4 = 8,
};

__host__ __device__ inline int qtype_block(int qt) {
  switch (qt) {
    case QT_Q8_0: case QT_Q4_0: return 32;
    case QT_Q4_K: case QT_Q5_K: case QT_Q6_K: return 256;
    case QT_NVFP4: return 64;
    default: return 1;
  }
}
__host__ __device__ inline int qtype_bytes(int qt) {
  switch (qt) {
    case QT_F32: return 4;
    case QT_F16: case QT_BF16: return 2;
    case QT_Q8_0: return 34;
    case QT_Q4_0: return 18;
    case QT_Q4_K: return 144;
    case QT_Q5_K: return 176;
    case QT_Q6_K: return 210;
    case QT_NVFP4: return 36;
    default: return 0;
  }
}

__device__ __forceinline__ float ld_f16(const uint8_t* p) {
  return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// 6-bit (scale, min) pair j of a Q4_K / Q5_K block from its 12 packed bytes
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& m) {
  if (j < 4) {
    sc = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// E2M1 magnitude table doubled (0, .5, 1, 1.5, 2, 3, 4, 6 times two); the scale decode carries the 0.5
__device__ __forceinline__ float e2m1_doubled(int code) {
  const int mag = code & 7;
  const float v = mag < 4 ? (float)mag : (mag == 4 ? 4.f : mag == 5 ? 6.f : mag == 6 ? 8.f : 12.f);
  return (code & 8) ? -v : v;
}
// NVFP4 sub-block scale byte (unsigned e4m3, bit 7 ignored), halved; 0x00 and 0x7F decode to 0
__device__ __forceinline__ float ue4m3_half(uint8_t b) {
  const int mag = b & 0x7F;
  if (mag == 0 || mag == 0x7F) return 0.f;
  const int e = mag >> 3, man = mag & 7;
  const float v = e == 0 ? ldexpf((float)man, -9) : ldexpf(1.f + (float)man * 0.125f, e - 7);
  return v * 0.5f;
}

// value `i` of a row encoded as `qt` (slow generic path: embedding rows, tests)
__device__ inline float dequant_elem(int qt, const uint8_t* row, int i) {
  switch (qt) {
    case QT_F32: return reinterpret_cast<const float*>(row)[i];
    case QT_F16: return __half2float(reinterpret_cast<const __half*>(row)[i]);
    case QT_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(row)[i]);
    case QT_Q8_0: {
      const uint8_t* b = row + (size_t)(i >> 5) * 34;
      return ld_f16(b) * (float)(int8_t)b[2 + (i & 31)];
    }
    case QT_Q4_0: {
      const uint8_t* b = row + (size_t)(i >> 5) * 18;
      const int j = i & 31;
      const int q = j < 16 ? (b[2 + j] & 0xF) : (b[2 + j - 16] >> 4);
      return ld_f16(b) * (float)(q - 8);
    }
    case QT_Q4_K: {
      const uint8_t* b = row + (size_t)(i >> 8) * 144;
      const int j = i & 255, sub = j >> 5, l = j & 31;
      int sc, m;
      scale_min_k4(sub, b + 4, sc, m);
      const uint8_t byte = b[16 + (sub >> 1) * 32 + l];
      const int q = (sub & 1) ? (byte >> 4) : (byte & 0xF);
      return ld_f16(b) * (float)sc * (float)q - ld_f16(b + 2) * (float)m;
    }
    case QT_Q5_K: {
      const uint8_t* b = row + (size_t)(i >> 8) * 176;
      const int j = i & 255, sub = j >> 5, l = j & 31;
      int sc, m;
      scale_min_k4(sub, b + 4, sc, m);
      const uint8_t byte = b[48 + (sub >> 1) * 32 + l];
      int q = (sub & 1) ? (byte >> 4) : (byte & 0xF);
      q += ((b[16 + l] >> sub) & 1) << 4;
      return ld_f16(b) * (float)sc * (float)q - ld_f16(b + 2) * (float)m;
    }
    case QT_Q6_K: {
      const uint8_t* b = row + (size_t)(i >> 8) * 210;
      const int j = i & 255, half = j >> 7, r = j & 127, quarter = r >> 5, l = r & 31;
      const uint8_t* ql = b + half * 64;
      const uint8_t* qh = b + 128 + half * 32;
      const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + half * 8;
      const uint8_t lo = ql[(quarter & 1) * 32 + l];
      const int q4 = (quarter & 2) ? (lo >> 4) : (lo & 0xF);
      const int q = (q4 | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
      return ld_f16(b + 208) * (float)sc[(l >> 4) + 2 * quarter] * (float)q;
    }
    case QT_NVFP4: {
      const uint8_t* b = row + (size_t)(i >> 6) * 36;
      const int j = i & 63, sub = j >> 4, l = j & 15;
      const uint8_t byte = b[4 + sub * 8 + (l & 7)];
      const int code = l < 8 ? (byte & 0xF) : (byte >> 4);
      return ue4m3_half(b[sub]) * e2m1_doubled(code);
    }
    default: return 0.f;
  }
}

}  // namespace oxb
