// Packed-weight GEMV for decode batches of 1..8 tokens: Y[T, N] = X[T, K] · dequant(Wq)[N, K]^T.
//
// At these batch sizes the projection is a pure stream of the packed weight bytes, and the tensor-core
// path (decode the blocks to bf16, stage them as UMMA tiles) spends more instructions per weight than
// the memory system needs time to deliver it.  This kernel keeps the weights packed all the way into the
// arithmetic: the activations are quantized once per CTA to int8 with one fp32 scale per 32 values
// (plus the integer sums that the offset terms of Q4_K / Q6_K / Q4_0 need), and every 4 weights cost one
// dp4a.  A persistent grid (CTAs = what the SMs hold) walks the rows, one warp per row pair, 8 lanes per
// 256-value super-block, 16-byte loads; per-row partial sums meet in a warp shuffle.
//
// Counterparts in the reference: gemv_q4k_q8kin_mw_kernel / gemv_q6k_* (oxidize-core/kernels/gemv_f32.cu:768)
// and k_mmq_matvec_* (oxidize-c/src/backends/cuda_mmq.cu); the block layouts are the GGUF ones
// (quant_blocks.cuh).
#pragma once
#include "common.cuh"
#include "quant_blocks.cuh"

namespace oxb {

constexpr int GV_WARPS = 8;
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_MAX_T = 8;

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {  // a unsigned bytes, b signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// 16 bytes from an address that is only 2-byte aligned: aligned words + funnel shift.
__device__ __forceinline__ void ld16_align2(const uint8_t* p, uint32_t (&o)[4]) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
  const uint32_t sh = (uint32_t)(a & 2) * 8;
  const uint32_t x0 = __ldg(w), x1 = __ldg(w + 1), x2 = __ldg(w + 2), x3 = __ldg(w + 3);
  const uint32_t x4 = sh ? __ldg(w + 4) : 0u;
  o[0] = __funnelshift_r(x0, x1, sh);
  o[1] = __funnelshift_r(x1, x2, sh);
  o[2] = __funnelshift_r(x2, x3, sh);
  o[3] = __funnelshift_r(x3, x4, sh);
}
__device__ __forceinline__ float ld_half_raw(const uint8_t* p) {
  return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p))));
}

// (scale, min) pair j of a Q4_K block whose 12 packed bytes are the words s0 s1 s2
__device__ __forceinline__ void scale_min_words(int j, uint32_t s0, uint32_t s1, uint32_t s2, int& sc, int& m) {
  const int sh = (j & 3) * 8;
  const uint32_t a = (s0 >> sh) & 0xFF, b = (s1 >> sh) & 0xFF, c = (s2 >> sh) & 0xFF;
  if (j < 4) {
    sc = a & 63;
    m = b & 63;
  } else {
    sc = (c & 0xF) | ((a >> 6) << 4);
    m = (c >> 4) | ((b >> 6) << 4);
  }
}

// Shared-memory view of the quantized activations of one CTA: for token t
//   q  [t*K + ...]      int8 codes, inside each 256-value super-block in the order of gv_act_pos
//   d  [t*K/32 + i/32]  fp32 scale of each 32-value block
//   s16[t*K/16 + i/16]  sum of the codes of each 16-value half block
struct GvAct {
  const int8_t* q;
  const float* d;
  const short* s16;
  int K;
};

// Position of activation value j (inside its 256-value super-block) in the shared-memory copy.  The k-quant layouts
// interleave their nibbles (a run of bytes holds values j.. in the low nibbles and j+32.. or j+64.. in the high ones), so
// with the activations in natural order the eight lanes that share a super-block would read 16-byte pieces that are
// 64 or 128 bytes apart and collide on the shared-memory banks.  The copy is therefore stored in the order in which
// the weight bytes ask for it: all "low nibble" partners of a super-block first (128 bytes, contiguous across the
// lanes), then all "high nibble" partners.
template <int QT>
__device__ __forceinline__ int gv_act_pos(int j) {
  if constexpr (QT == QT_Q4_K) {
    const int c = j >> 6, r = j & 63;           // group of 64 values: 32 low-nibble, then 32 high-nibble ones
    return r < 32 ? 32 * c + r : 128 + 32 * c + (r - 32);
  } else if constexpr (QT == QT_Q6_K) {
    const int h = j >> 7, r = j & 127;          // half of 128 values: 64 low-nibble, then 64 high-nibble ones
    return r < 64 ? 64 * h + r : 128 + 64 * h + (r - 64);
  } else {
    return j;
  }
}

// Values of one row covered by one warp iteration, per format.
template <int QT>
struct GvSpan {
  static constexpr int VALUES = (QT == QT_Q4_K || QT == QT_Q6_K) ? 1024 : (QT == QT_Q8_0 ? 512 : 1024);
};

// The packed words one lane needs for its share of one warp iteration of one row.  Loading them (gv_load) is kept
// apart from using them (gv_dot) so that the loads of several iterations and rows are in flight together: at decode
// sizes a warp sees only a handful of iterations per row, and a load-use-load-use chain would leave the kernel
// waiting on one memory latency after the other.
template <int QT>
struct GvFrag {
  uint32_t a[4];   // Q4_K: header words (d|dmin, 12 scale bytes)   Q6_K: ql   Q8_0 / Q4_0: codes
  uint32_t b[4];   // Q4_K: 16 bytes of nibbles                     Q6_K: qh
  float d, dlo, dhi;  // Q6_K: d * sub-block scales; Q8_0 / Q4_0: block scale in d
  bool live;
};

template <int QT>
__device__ __forceinline__ void gv_load(const uint8_t* rowp, int it, int lane, int K, GvFrag<QT>& f) {
  f.live = false;
  if constexpr (QT == QT_Q4_K) {
    const int sb = it * 4 + (lane >> 3);
    if (sb * 256 >= K) return;
    const int l8 = lane & 7;
    const uint8_t* b = rowp + (size_t)sb * 144;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(b));
    const uint4 qv = __ldg(reinterpret_cast<const uint4*>(b + 16 + 16 * l8));
    f.a[0] = hdr.x; f.a[1] = hdr.y; f.a[2] = hdr.z; f.a[3] = hdr.w;
    f.b[0] = qv.x; f.b[1] = qv.y; f.b[2] = qv.z; f.b[3] = qv.w;
    f.live = true;
  } else if constexpr (QT == QT_Q6_K) {
    const int sb = it * 4 + (lane >> 3);
    if (sb * 256 >= K) return;
    const int l8 = lane & 7, h = l8 >> 2, i = l8 & 3, q0 = i >> 1, lr = (i & 1) * 16;
    const uint8_t* b = rowp + (size_t)sb * 210;
    ld16_align2(b + h * 64 + 16 * i, f.a);
    ld16_align2(b + 128 + h * 32 + lr, f.b);
    const int8_t* scp = reinterpret_cast<const int8_t*>(b + 192) + h * 8 + (i & 1) + 2 * q0;
    const float d = ld_half_raw(b + 208);
    f.dlo = d * (float)__ldg(scp);
    f.dhi = d * (float)__ldg(scp + 4);
    f.live = true;
  } else if constexpr (QT == QT_Q8_0) {
    const int blk = it * 16 + (lane >> 1), hh = lane & 1;
    if (blk * 32 >= K) return;
    const uint8_t* b = rowp + (size_t)blk * 34;
    ld16_align2(b + 2 + 16 * hh, f.a);
    f.d = ld_half_raw(b);
    f.live = true;
  } else if constexpr (QT == QT_Q4_0) {
    const int blk = it * 32 + lane;
    if (blk * 32 >= K) return;
    const uint8_t* b = rowp + (size_t)blk * 18;
    ld16_align2(b + 2, f.a);
    f.d = ld_half_raw(b);
    f.live = true;
  }
}

// One lane's share of one warp iteration of one row: adds the contribution to each token's sum.
template <int QT, int TB>
__device__ __forceinline__ void gv_dot(const GvFrag<QT>& f, int it, int lane, const GvAct& act, float (&acc)[TB]) {
  if (!f.live) return;
  if constexpr (QT == QT_Q4_K) {
    const int sb = it * 4 + (lane >> 3);
    const int l8 = lane & 7, c = l8 >> 1, hh = l8 & 1;
    const float d = __half2float(__ushort_as_half((unsigned short)(f.a[0] & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(f.a[0] >> 16)));
    int sc0, m0, sc1, m1;
    scale_min_words(2 * c, f.a[1], f.a[2], f.a[3], sc0, m0);
    scale_min_words(2 * c + 1, f.a[1], f.a[2], f.a[3], sc1, m1);
    const float ds0 = d * (float)sc0, dm0 = dmin * (float)m0, ds1 = d * (float)sc1, dm1 = dmin * (float)m1;
    const int off = sb * 256 + 64 * c + 16 * hh;  // first value of the low-nibble run; the high-nibble run is 32 further
    const int xoff = sb * 256 + 16 * l8;          // where those runs sit in the permuted copy (gv_act_pos); high: + 128
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int8_t* xq = act.q + (size_t)t * act.K + xoff;
      const uint4 xl = *reinterpret_cast<const uint4*>(xq);
      const uint4 xh = *reinterpret_cast<const uint4*>(xq + 128);
      const uint32_t xlw[4] = {xl.x, xl.y, xl.z, xl.w}, xhw[4] = {xh.x, xh.y, xh.z, xh.w};
      int slo = 0, shi = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        slo = dp4a_ss(f.b[w] & 0x0F0F0F0Fu, xlw[w], slo);
        shi = dp4a_ss((f.b[w] >> 4) & 0x0F0F0F0Fu, xhw[w], shi);
      }
      const float* dx = act.d + (size_t)t * (act.K >> 5) + (off >> 5);
      const short* s16 = act.s16 + (size_t)t * (act.K >> 4) + (off >> 4);
      acc[t] += dx[0] * (ds0 * (float)slo - dm0 * (float)s16[0]) + dx[1] * (ds1 * (float)shi - dm1 * (float)s16[2]);
    }
  } else if constexpr (QT == QT_Q6_K) {
    const int sb = it * 4 + (lane >> 3);
    const int l8 = lane & 7, h = l8 >> 2, i = l8 & 3, q0 = i >> 1, lr = (i & 1) * 16;
    uint32_t vlo[4], vhi[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      vlo[w] = (f.a[w] & 0x0F0F0F0Fu) | (((f.b[w] >> (2 * q0)) & 0x03030303u) << 4);
      vhi[w] = ((f.a[w] >> 4) & 0x0F0F0F0Fu) | (((f.b[w] >> (2 * q0 + 4)) & 0x03030303u) << 4);
    }
    const int off = sb * 256 + h * 128 + q0 * 32 + lr;  // low-nibble run; the high-nibble run is 64 further
    const int xoff = sb * 256 + 16 * l8;                // in the permuted copy (gv_act_pos); high: + 128
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int8_t* xq = act.q + (size_t)t * act.K + xoff;
      const uint4 xl = *reinterpret_cast<const uint4*>(xq);
      const uint4 xh = *reinterpret_cast<const uint4*>(xq + 128);
      const uint32_t xlw[4] = {xl.x, xl.y, xl.z, xl.w}, xhw[4] = {xh.x, xh.y, xh.z, xh.w};
      int slo = 0, shi = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        slo = dp4a_us(vlo[w], xlw[w], slo);
        shi = dp4a_us(vhi[w], xhw[w], shi);
      }
      const float* dx = act.d + (size_t)t * (act.K >> 5) + (off >> 5);
      const short* s16 = act.s16 + (size_t)t * (act.K >> 4) + (off >> 4);
      acc[t] += f.dlo * dx[0] * (float)(slo - 32 * (int)s16[0]) + f.dhi * dx[2] * (float)(shi - 32 * (int)s16[4]);
    }
  } else if constexpr (QT == QT_Q8_0) {
    const int blk = it * 16 + (lane >> 1), hh = lane & 1;
    const int off = blk * 32 + 16 * hh;
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const uint4 xv = *reinterpret_cast<const uint4*>(act.q + (size_t)t * act.K + off);
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      int s = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) s = dp4a_ss(f.a[w], xw[w], s);
      acc[t] += f.d * act.d[(size_t)t * (act.K >> 5) + blk] * (float)s;
    }
  } else if constexpr (QT == QT_Q4_0) {
    const int blk = it * 32 + lane;
    const int off = blk * 32;
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int8_t* xq = act.q + (size_t)t * act.K + off;
      const uint4 xl = *reinterpret_cast<const uint4*>(xq);
      const uint4 xh = *reinterpret_cast<const uint4*>(xq + 16);
      const uint32_t xlw[4] = {xl.x, xl.y, xl.z, xl.w}, xhw[4] = {xh.x, xh.y, xh.z, xh.w};
      int s = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        s = dp4a_ss(f.a[w] & 0x0F0F0F0Fu, xlw[w], s);
        s = dp4a_ss((f.a[w] >> 4) & 0x0F0F0F0Fu, xhw[w], s);
      }
      const short* s16 = act.s16 + (size_t)t * (act.K >> 4) + (off >> 4);
      acc[t] += f.d * act.d[(size_t)t * (act.K >> 5) + blk] * (float)(s - 8 * ((int)s16[0] + (int)s16[1]));
    }
  }
}

// Quantize X[T, K] (bf16, row stride ldX) into the CTA's shared memory: int8 codes, a scale per 32 values,
// the code sum per 16 values.  Rows t >= T are zero.  Every thread of the CTA takes part.
template <int QT, int TB>
__device__ __forceinline__ void gv_quantize_x(const __nv_bfloat16* __restrict__ X, int ldX, int T, int K, int8_t* q, float* d,
                                              short* s16) {
  const int chunks = K >> 3;  // 8 values per thread-step; 4 consecutive lanes share one 32-value block
  const int total = TB * chunks;
  for (int base = 0; base < total; base += blockDim.x) {
    const int idx = base + threadIdx.x;
    const bool live = idx < total;
    const int t = live ? idx / chunks : 0, ch = live ? idx - t * chunks : 0;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (live && t < T) {
      const uint4 raw = *reinterpret_cast<const uint4*>(X + (size_t)t * ldX + ch * 8);
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(rw[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float scale = amax / 127.f;
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    int qi[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      qi[j] = __float2int_rn(v[j] * inv);
      sum += qi[j];
    }
    const int pair = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
    if (live) {
      const uint32_t w0 = (qi[0] & 0xFF) | ((qi[1] & 0xFF) << 8) | ((qi[2] & 0xFF) << 16) | ((uint32_t)(qi[3] & 0xFF) << 24);
      const uint32_t w1 = (qi[4] & 0xFF) | ((qi[5] & 0xFF) << 8) | ((qi[6] & 0xFF) << 16) | ((uint32_t)(qi[7] & 0xFF) << 24);
      // (8 consecutive values stay consecutive under gv_act_pos)
      const int j = ch * 8;
      *reinterpret_cast<uint2*>(q + (size_t)t * K + (j & ~255) + gv_act_pos<QT>(j & 255)) = make_uint2(w0, w1);
      if ((ch & 1) == 0) s16[(size_t)t * (K >> 4) + (ch >> 1)] = (short)pair;
      if ((ch & 3) == 0) d[(size_t)t * (K >> 5) + (ch >> 2)] = scale;
    }
  }
}

// Shared-memory bytes of the quantized activations for TB tokens of K values
__host__ __device__ inline size_t gv_smem_bytes(int TB, int K) { return (size_t)TB * ((size_t)K + (size_t)(K >> 5) * 4 + (size_t)(K >> 4) * 2); }

template <int QT, int TB, int RPW>
__global__ void __launch_bounds__(GV_THREADS)
gemv_quant_kernel(const uint8_t* __restrict__ W, size_t row_bytes, const __nv_bfloat16* __restrict__ X, int ldX,
                  __nv_bfloat16* __restrict__ Y, int ldY, const float* __restrict__ bias, int T, int N, int K, int add_into) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  int8_t* xq = reinterpret_cast<int8_t*>(gv_smem);
  float* xd = reinterpret_cast<float*>(gv_smem + (size_t)TB * K);
  short* xs = reinterpret_cast<short*>(gv_smem + (size_t)TB * K + (size_t)TB * (K >> 5) * 4);
  pdl_launch_dependents();
  pdl_wait();  // the activations come from the upstream kernel
  gv_quantize_x<QT, TB>(X, ldX, T, K, xq, xd, xs);
  __syncthreads();
  const GvAct act{xq, xd, xs, K};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * GV_WARPS + warp, nw = gridDim.x * GV_WARPS;
  const int iters = (K + GvSpan<QT>::VALUES - 1) / GvSpan<QT>::VALUES;
  for (int r0 = gw * RPW; r0 < N; r0 += nw * RPW) {
    float acc[RPW][TB];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int t = 0; t < TB; ++t) acc[r][t] = 0.f;
    // iterations in groups of G: all loads of a group (G iterations x RPW rows) are issued before the first use
    constexpr int G = 2;
    for (int it0 = 0; it0 < iters; it0 += G) {
      GvFrag<QT> fr[G][RPW];
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const int row = r0 + r < N ? r0 + r : N - 1;  // a clamped row is computed and dropped
          if (it0 + g < iters) gv_load<QT>(W + (size_t)row * row_bytes, it0 + g, lane, K, fr[g][r]);
          else fr[g][r].live = false;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) gv_dot<QT, TB>(fr[g][r], it0 + g, lane, act, acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        float v = warp_sum(acc[r][t]);
        if (lane == 0 && r0 + r < N && t < T) {
          if (bias != nullptr) v += bias[r0 + r];
          __nv_bfloat16* dst = Y + (size_t)t * ldY + r0 + r;
          if (add_into) v += __bfloat162float(*dst);
          *dst = __float2bfloat16(v);
        }
      }
    }
  }
}

template <int QT, int TB>
int gemv_quant_launch(const uint8_t* W, size_t row_bytes, const __nv_bfloat16* X, int ldX, __nv_bfloat16* Y, int ldY,
                      const float* bias, int T, int N, int K, int add_into, int sm_count, cudaStream_t stream) {
  constexpr int RPW = TB <= 2 ? 2 : 1;
  const size_t smem = gv_smem_bytes(TB, K);
  auto kfn = gemv_quant_kernel<QT, TB, RPW>;
  static size_t configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (smem > 48 * 1024 && smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = smem;
  }
  int per_sm = (int)((200 * 1024) / (smem + 1024));
  if (per_sm > 4) per_sm = 4;
  if (per_sm < 1) per_sm = 1;
  int grid = (N + GV_WARPS * RPW - 1) / (GV_WARPS * RPW);
  if (grid > sm_count * per_sm) grid = sm_count * per_sm;
  cudaError_t le = oxb_launch(kfn, dim3(grid), dim3(GV_THREADS), smem, stream, W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into);
  if (le != cudaSuccess) return (int)le;
  OXB_CHECK_LAUNCH();
  return 0;
}

// Whether the GEMV covers this call: format, batch, shape and alignment.
inline bool gemv_quant_supported(int qtype, int T, int K, size_t row_bytes, const void* W, const void* X, int ldX) {
  if (T < 1 || T > GV_MAX_T) return false;
  if (!(qtype == QT_Q4_K || qtype == QT_Q6_K || qtype == QT_Q8_0 || qtype == QT_Q4_0)) return false;
  if (K % qtype_block(qtype) != 0 || K % 32 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(X) & 15) != 0 || ldX % 8 != 0) return false;
  if (qtype == QT_Q4_K && ((reinterpret_cast<uintptr_t>(W) & 15) != 0 || row_bytes % 16 != 0)) return false;
  if ((reinterpret_cast<uintptr_t>(W) & 1) != 0 || row_bytes % 2 != 0) return false;
  const int tb = T <= 1 ? 1 : T <= 2 ? 2 : T <= 4 ? 4 : 8;
  return gv_smem_bytes(tb, K) <= 200 * 1024;
}

template <int QT>
int gemv_quant_dispatch_t(const uint8_t* W, size_t row_bytes, const __nv_bfloat16* X, int ldX, __nv_bfloat16* Y, int ldY,
                          const float* bias, int T, int N, int K, int add_into, int sm_count, cudaStream_t stream) {
  if (T <= 1) return gemv_quant_launch<QT, 1>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
  if (T <= 2) return gemv_quant_launch<QT, 2>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
  if (T <= 4) return gemv_quant_launch<QT, 4>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
  return gemv_quant_launch<QT, 8>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
}

inline int gemv_quant(int qtype, const uint8_t* W, size_t row_bytes, const __nv_bfloat16* X, int ldX, __nv_bfloat16* Y, int ldY,
                      const float* bias, int T, int N, int K, int add_into, int sm_count, cudaStream_t stream) {
  switch (qtype) {
    case QT_Q4_K: return gemv_quant_dispatch_t<QT_Q4_K>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
    case QT_Q6_K: return gemv_quant_dispatch_t<QT_Q6_K>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
    case QT_Q8_0: return gemv_quant_dispatch_t<QT_Q8_0>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
    case QT_Q4_0: return gemv_quant_dispatch_t<QT_Q4_0>(W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace oxb
