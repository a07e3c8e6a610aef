// Memory-bound glue kernels: embedding gather (dense or block-quantized table), fused
// residual-add + RMSNorm, SwiGLU, fused QK-norm + RoPE + paged-KV write (bf16/f16/q8/q4),
// and greedy argmax.  Each fuses what the reference runs as separate launches
// (oxidize-core/kernels/gemv_f32.cu: rms_norm :1680, residual_add :1720, silu_mul :1738,
// rope :1928, kv_append :1990, embed :2258/:2271; oxidize-c k_residual_rms cuda.cu:561,
// k_qk_norm_rope cuda_qwen35.cu:46, k_f_argmax cuda_fast.cu:495).
#pragma once
#include "common.cuh"
#include "quant_blocks.cuh"

namespace oxb {

// ----------------------------------------------------------------------------- embedding
// one CTA per token; qtype as in quant_blocks.cuh
static __global__ void embed_kernel(const int* __restrict__ tokens, const uint8_t* __restrict__ table, int qtype,
                             size_t row_bytes, int H, int vocab, float scale, __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) tok = 0;
  const uint8_t* row = table + (size_t)tok * row_bytes;
  __nv_bfloat16* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = __float2bfloat16(dequant_elem(qtype, row, i) * scale);
}

// ----------------------------------------------------------------------------- add + RMSNorm
// y = rmsnorm(x + residual) * w ; residual <- x + residual (bf16, rounded before the norm)
// one CTA per row; the summed row is staged in shared memory as fp32.
static __global__ void add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res_in,
                                   __nv_bfloat16* __restrict__ res_out, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, int H, float eps) {
  extern __shared__ float rowbuf[];
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  const int H8 = H >> 3;
  for (int i = threadIdx.x; i < H8; i += blockDim.x) {
    uint4 xv = *reinterpret_cast<const uint4*>(x + base + i * 8);
    uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(xs[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
    if (res_in != nullptr) {
      uint4 rv = *reinterpret_cast<const uint4*>(res_in + base + i * 8);
      uint32_t rs[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(rs[j]);
        v[2 * j] += f.x;
        v[2 * j + 1] += f.y;
      }
    }
    uint4 ov;
    uint32_t* os = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      os[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
      float2 f = unpack_bf16x2(os[j]);  // the norm sees the rounded residual
      rowbuf[i * 8 + 2 * j] = f.x;
      rowbuf[i * 8 + 2 * j + 1] = f.y;
      ss += f.x * f.x + f.y * f.y;
    }
    if (res_out != nullptr) *reinterpret_cast<uint4*>(res_out + base + i * 8) = ov;
  }
  for (int i = H8 * 8 + threadIdx.x; i < H; i += blockDim.x) {  // tail when H % 8 != 0
    float v = __bfloat162float(x[base + i]);
    if (res_in != nullptr) v += __bfloat162float(res_in[base + i]);
    __nv_bfloat16 r = __float2bfloat16(v);
    if (res_out != nullptr) res_out[base + i] = r;
    v = __bfloat162float(r);
    rowbuf[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float inv = rsqrtf(total / (float)H + eps);
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) y[base + i] = __float2bfloat16(rowbuf[i] * inv * w[i]);
}

// Register-resident variant for H % 8 == 0 and H <= 8 * CH * 1024: every thread owns CH 16-byte
// chunks of the row, the norm weights are fetched before the reduction so that only one memory
// round trip sits in front of the block-wide sum, and nothing is staged in shared memory.
template <int CH>
__global__ void __launch_bounds__(1024)
add_rmsnorm_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res_in,
                       __nv_bfloat16* __restrict__ res_out, const float* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, int H, float eps) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * H;
  const int H8 = H >> 3;
  float v[CH][8];
  float4 w0[CH], w1[CH];
  float ss = 0.f;
  pdl_launch_dependents();
  // the norm weights are static: fetch them before waiting for the upstream kernel
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < H8) {
      w0[c] = *reinterpret_cast<const float4*>(w + i * 8);
      w1[c] = *reinterpret_cast<const float4*>(w + i * 8 + 4);
    }
  }
  pdl_wait();
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < H8) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x + base + i * 8);
      uint4 rv = make_uint4(0, 0, 0, 0);
      if (res_in != nullptr) rv = *reinterpret_cast<const uint4*>(res_in + base + i * 8);
      const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, rs[4] = {rv.x, rv.y, rv.z, rv.w};
      uint4 ov;
      uint32_t* os = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = unpack_bf16x2(xs[j]), b = unpack_bf16x2(rs[j]);
        os[j] = pack_bf16x2(a.x + b.x, a.y + b.y);
        const float2 f = unpack_bf16x2(os[j]);  // the norm sees the rounded residual
        v[c][2 * j] = f.x;
        v[c][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      if (res_out != nullptr) *reinterpret_cast<uint4*>(res_out + base + i * 8) = ov;
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < H8) {
      const float ww[8] = {w0[c].x, w0[c].y, w0[c].z, w0[c].w, w1[c].x, w1[c].y, w1[c].z, w1[c].w};
      uint4 ov;
      uint32_t* os = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) os[j] = pack_bf16x2(v[c][2 * j] * inv * ww[2 * j], v[c][2 * j + 1] * inv * ww[2 * j + 1]);
      *reinterpret_cast<uint4*>(y + base + i * 8) = ov;
    }
  }
}

// ----------------------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, I + i]
// Sum of squares of every row of X[T, H] (bf16) as 64-bit fixed point (2^-28 units): seeds the folded RMSNorm of
// the first layer (later layers get these sums from the epilogue that writes the residual stream).  One warp per row.
static __global__ void row_sumsq_kernel(const __nv_bfloat16* __restrict__ X, int ldX, int T, int H,
                                        unsigned long long* __restrict__ out, unsigned long long* __restrict__ clear) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  // per 128-column tile, as the GEMM epilogues do, so that both routes round alike
  unsigned long long total = 0ull;
  for (int c0 = 0; c0 < H; c0 += 256) {
    const int c = c0 + lane * 8;
    float s = 0.f;
    if (c < H) {
      const uint4 v = *reinterpret_cast<const uint4*>(X + (size_t)t * ldX + c);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]);
        s += f.x * f.x + f.y * f.y;
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float other = __shfl_xor_sync(0xffffffffu, s, 16);
    if (lane == 0) {
      total += (unsigned long long)(fminf(s, 3.0e10f) * 268435456.f + 0.5f);
      if (c0 + 128 < H) total += (unsigned long long)(fminf(other, 3.0e10f) * 268435456.f + 0.5f);
    }
  }
  if (lane == 0) {  // accumulators of neighbouring tokens are 16 words (128 bytes) apart, see NormArgs
    out[(size_t)t * 16] = total;
    if (clear != nullptr) clear[(size_t)t * 16] = 0ull;
  }
}

// act(gate) * up over the two halves of a fused [T, 2I] projection.  GELU = false: SiLU (SwiGLU); true: the tanh form of
// GELU (GeGLU, Gemma): 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) = g * sigmoid(2 sqrt(2/pi) (g + 0.044715 g^3)).
template <bool GELU>
static __device__ __forceinline__ float gated_act(float g) {
  const float z = GELU ? 1.5957691216057308f * (g + 0.044715f * g * g * g) : g;
  return g / (1.f + __expf(-z));
}

template <bool GELU>
static __global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int T, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const int I8 = I >> 3;
  const size_t total = (size_t)T * I8;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I8;
    const int i = (int)(idx % I8) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * I + i);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + i);
    const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
    uint4 o;
    uint32_t* os = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(gs[j]), b = unpack_bf16x2(us[j]);
      os[j] = pack_bf16x2(gated_act<GELU>(a.x) * b.x, gated_act<GELU>(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = o;
  }
}

// ----------------------------------------------------------------------------- QK-norm + RoPE + KV write
// grid (T, nq + 2*nkv), block = head_dim threads.  Head h < nq: query (norm, rope, store to q_out);
// nq <= h < nq+nkv: key (norm, rope, write to cache); else value (write to cache).
// cos_sin: [max_pos, rot] fp32 (cos for pair i at [p, i], sin at [p, rot/2 + i]).
// KV cache layout: [block, kv_head, 2, page, head_dim(/2 for q4)]; scales [block, kv_head, 2, page, hd/32].
struct KvWriteArgs {
  void* kv_data;
  float* kv_scales;
  int kv_mode;  // 0 bf16, 1 f16, 2 q8, 3 q4, 4 f32
  int page;
  int nkv;
  int num_blocks;  // pages in the KV pool: slots are checked against it
};

static __global__ void qk_rope_kvwrite_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                       const int* __restrict__ slots, const float* __restrict__ cos_sin, int max_pos,
                                       int rot, int pairing /*0 split-half, 1 adjacent*/, const float* __restrict__ qn,
                                       const float* __restrict__ kn, float eps, int nq, int nkv, int hd,
                                       __nv_bfloat16* __restrict__ q_out, KvWriteArgs kv) {
  extern __shared__ float hbuf[];  // hd floats
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int width = (nq + 2 * nkv) * hd;
  float v = __bfloat162float(qkv[(size_t)t * width + (size_t)h * hd + d]);
  const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
  if (is_q || is_k) {
    const float* nw = is_q ? qn : kn;
    if (nw != nullptr) {
      const float ss = block_sum(v * v, red);
      v = v * rsqrtf(ss / (float)hd + eps) * nw[d];
    }
    hbuf[d] = v;
    __syncthreads();
    if (d < rot) {
      int p = positions[t];
      p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
      const int half = rot >> 1;
      int pair, partner;
      bool first;
      if (pairing == 0) {
        first = d < half;
        pair = first ? d : d - half;
        partner = first ? d + half : d - half;
      } else {
        first = (d & 1) == 0;
        pair = d >> 1;
        partner = d ^ 1;
      }
      const float c = cos_sin[(size_t)p * rot + pair], s = cos_sin[(size_t)p * rot + half + pair];
      const float o = hbuf[partner];
      v = first ? (v * c - o * s) : (v * c + o * s);
    }
  }
  if (is_q) {
    q_out[((size_t)t * nq + h) * hd + d] = __float2bfloat16(v);
    return;
  }
  const int slot = slots[t];
  if (slot < 0) return;
  const int kvh = is_k ? h - nq : h - nq - nkv;
  const int which = is_k ? 0 : 1;
  const int blk = slot / kv.page, off = slot % kv.page;
  if (blk >= kv.num_blocks) {  // never write outside the pool: record the slot and skip
    if (d == 0) oxb_report(OXB_BAD_SLOT, slot);
    return;
  }
  const size_t row = (((size_t)blk * kv.nkv + kvh) * 2 + which) * kv.page + off;
  if (kv.kv_mode == 0) {
    reinterpret_cast<__nv_bfloat16*>(kv.kv_data)[row * hd + d] = __float2bfloat16(v);
  } else if (kv.kv_mode == 1) {
    reinterpret_cast<__half*>(kv.kv_data)[row * hd + d] = __float2half(v);
  } else if (kv.kv_mode == 4) {
    reinterpret_cast<float*>(kv.kv_data)[row * hd + d] = v;
  } else {
    // symmetric per-32-channel blocks; one warp == one block (hd is a multiple of 32)
    const float qmax = kv.kv_mode == 2 ? 127.f : 7.f;
    const float amax = warp_max(fabsf(v));
    const float scale = amax / qmax;
    const float inv = scale > 0.f ? 1.f / scale : 0.f;
    const int q = (int)fminf(fmaxf(rintf(v * inv), -qmax), qmax) + (int)qmax;
    if ((d & 31) == 0) kv.kv_scales[row * (hd >> 5) + (d >> 5)] = scale;
    uint8_t* data = reinterpret_cast<uint8_t*>(kv.kv_data);
    if (kv.kv_mode == 2) {
      data[row * hd + d] = (uint8_t)q;
    } else {
      const int hi = __shfl_down_sync(0xffffffffu, q, 1);
      if ((d & 1) == 0) data[row * (hd >> 1) + (d >> 1)] = (uint8_t)(q | (hi << 4));
    }
  }
}

// ----------------------------------------------------------------------------- argmax
// one CTA per row of fp32 logits; tie_highest selects the last maximal index
static __global__ void argmax_kernel(const float* __restrict__ logits, int V, int ld, int tie_highest, int* __restrict__ out,
                              float* __restrict__ out_val, int index_offset) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = -1;  // -1 = nothing seen yet
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    // per-thread indices increase, so on ties the later one wins only under tie_highest
    if (bi < 0 || v > best || (v == best && tie_highest)) {
      if (!(v != v)) {
        best = v;
        bi = i;
      }
    }
  }
  auto better = [&](float v, int i, float bv, int b) {
    if (i < 0) return false;
    if (b < 0) return true;
    return v > bv || (v == bv && (tie_highest ? i > b : i < b));
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      if (bi < 0) bi = 0;  // all-NaN row
      out[blockIdx.x] = bi + index_offset;
      if (out_val != nullptr) out_val[blockIdx.x] = best;
    }
  }
}

// ----------------------------------------------------------------------------- vocabulary-parallel argmax
// Greedy sampling over a vocabulary that is sharded across tensor-parallel ranks, in ONE kernel: every rank
// reduces its own logits shard to a (value, index) pair per row, pushes the pair into every peer's exchange
// buffer over NVLink (8-byte words {payload, epoch}: a word that carries this call's epoch also carries its
// payload, so no fence or separate flag is needed), waits (bounded) for the pairs of the other ranks and picks the
// winner.  Shards are in ascending vocabulary order, so the first maximum is the lowest index and the last one
// the highest.  All ranks obtain the same token.  The token can be written to a second array as well (the next
// step's input ids, so that decode never needs the host to feed the token back).
// Replaces the reference's k_f_argmax + host feedback (oxidize-c/src/backends/cuda_fast.cu:495) for the sharded case.
struct ArgmaxXchg {
  int world, rank;                        // world <= 1: no exchange
  unsigned long long* bufs[8];            // peers' buffers: [2 parities][world][rmax][2] u64
  int* ctrl;                              // local: [0] call counter, [1] rows done
  int rmax;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename TIn>
static __global__ void __launch_bounds__(1024)
argmax_tp_kernel(const TIn* __restrict__ logits, int V, int ld, int tie_highest, int* __restrict__ out, int* __restrict__ out2,
                 int index_offset, const ArgmaxXchg xa) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cand_v[8];
  __shared__ int cand_i[8];
  __shared__ int s_call, s_fail;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    s_call = xa.world > 1 ? *reinterpret_cast<volatile int*>(xa.ctrl) : 0;
    s_fail = 0;
  }
  const TIn* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = (float)row[i];
    if (bi < 0 || v > best || (v == best && tie_highest)) {
      if (!(v != v)) {
        best = v;
        bi = i;
      }
    }
  }
  auto better = [&](float v, int i, float bv, int b) {
    if (i < 0) return false;
    if (b < 0) return true;
    return v > bv || (v == bv && (tie_highest ? i > b : i < b));
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (bi < 0) {  // all-NaN shard
      bi = 0;
      best = -INFINITY;
    }
    bi += index_offset;
    if (xa.world > 1) {
      const unsigned epoch = (unsigned)s_call + 1u != 0u ? (unsigned)s_call + 1u : 1u;
      const size_t par = (size_t)(s_call & 1) * xa.world;
      const int r = blockIdx.x;
      if (lane < xa.world) {
        // push this rank's pair to peer `lane` (self included)
        volatile unsigned long long* dst = xa.bufs[lane] + ((par + xa.rank) * xa.rmax + r) * 2;
        dst[0] = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(best);
        dst[1] = ((unsigned long long)epoch << 32) | (unsigned long long)(unsigned)bi;
        // wait for the pair of source rank `lane`
        volatile unsigned long long* src = xa.bufs[xa.rank] + ((par + lane) * xa.rmax + r) * 2;
        const unsigned long long t0 = gtimer_ns();
        unsigned long long w0 = 0ull, w1 = 0ull;
        bool got = false;
        for (unsigned it = 0;; ++it) {
          w0 = src[0];
          w1 = src[1];
          if ((unsigned)(w0 >> 32) == epoch && (unsigned)(w1 >> 32) == epoch) {
            got = true;
            break;
          }
          if ((it & 63u) == 63u && gtimer_ns() - t0 > xa.timeout_ns) break;
        }
        if (got) {
          cand_v[lane] = __uint_as_float((unsigned)(w0 & 0xFFFFFFFFull));
          cand_i[lane] = (int)(unsigned)(w1 & 0xFFFFFFFFull);
        } else {
          cand_v[lane] = -INFINITY;
          cand_i[lane] = 0;
          s_fail = 1;
          oxb_report(OXB_TIMEOUT_PEER_FLAG, lane);
        }
      }
      __syncwarp();
      if (lane == 0) {
        float wv = cand_v[0];
        int wi = cand_i[0];
        for (int s = 1; s < xa.world; ++s) {
          const float v = cand_v[s];
          if (v > wv || (v == wv && tie_highest)) {
            wv = v;
            wi = cand_i[s];
          }
        }
        bi = wi;
      }
    }
    if (lane == 0) {
      out[blockIdx.x] = bi;
      if (out2 != nullptr) out2[blockIdx.x] = bi;
      if (xa.world > 1) {
        // the last row of the grid advances the call counter (flips the buffer parity)
        __threadfence();
        if (atomicAdd(&xa.ctrl[1], 1) == (int)gridDim.x - 1) {
          xa.ctrl[1] = 0;
          __threadfence();
          xa.ctrl[0] = s_call + 1;
        }
      }
    }
  }
}

}  // namespace oxb
