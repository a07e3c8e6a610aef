// Mixture-of-experts routing and combine.
//
// moe_route_kernel: one warp per token.  Router logits -> softmax or sigmoid(+selection bias)
// -> top-k (lowest expert index wins ties) -> optional renormalisation -> scale; writes the
// (expert id, weight) pairs AND, for the experts held by this rank, a dense per-expert weight row
// scale[e_local][t] (0 where the token is not routed to e).  The grouped expert GEMM reads that row
// to skip idle experts, and the combine kernel uses it for the weighted sum, so no token lists,
// sorting or host round trip are needed and the whole MoE layer can be captured in a CUDA graph.
//
// moe_combine_kernel: out[t] = sum_e scale[e][t] * y[e][t] (+ shared-expert output), i.e. the top-k
// weighted sum fused with the shared-expert add.
//
// Semantics follow moe_ffn_forward_weights (oxidize-core/src/model/inference.rs:1690-1804,1852-1857);
// the reference routes on the device with k_moe_route<<<1,1>>> (oxidize-c/src/backends/cuda.cu:495).
#pragma once
#include "common.cuh"
#include "comm_fused.cuh"

namespace oxb {

constexpr int MOE_MAX_EXPERTS = 256;  // 8 logits per lane
constexpr int MOE_MAX_TOPK = 16;

// logits [T, E] fp32 (row stride ld); ids/wts [T, k]; scale [n_local, scale_ld] (may be null)
static __global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int ld, int k, int sigmoid,
                                 const float* __restrict__ sel_bias, int renorm, float weight_scale,
                                 int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ scale,
                                 int scale_ld, int first_local, int n_local, int n_groups, int groups_used) {
  __shared__ float s_sel[4][MOE_MAX_EXPERTS];  // launch uses 4 warps per block
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const float* row = logits + (size_t)t * ld;
  constexpr int PER = MOE_MAX_EXPERTS / 32;
  float score[PER], sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    score[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, score[j]);
  }
  if (sigmoid) {
#pragma unroll
    for (int j = 0; j < PER; ++j) score[j] = (lane + 32 * j) < E ? 1.f / (1.f + __expf(-score[j])) : 0.f;
  } else {
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      score[j] = (lane + 32 * j) < E ? __expf(score[j] - mx) : 0.f;
      s += score[j];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < PER; ++j) score[j] *= inv;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    sel[j] = e < E ? score[j] + (sel_bias != nullptr ? sel_bias[e] : 0.f) : -INFINITY;
  }
  if (n_groups > 1 && groups_used > 0) {
    // group-limited routing (DeepSeek): experts form n_groups (<= 32) contiguous groups; only the
    // groups_used best groups stay eligible.  Group score = sum of the two best biased scores when a
    // selection bias exists, else the best score.  Lane g scores group g from the warp's row in shared memory.
    float* row_sel = s_sel[threadIdx.x >> 5];
#pragma unroll
    for (int j = 0; j < PER; ++j) row_sel[lane + 32 * j] = sel[j];
    __syncwarp();
    const int gs = E / n_groups;
    float gscore = -INFINITY;
    if (lane < n_groups) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int i = 0; i < gs; ++i) {
        const float v = row_sel[lane * gs + i];
        if (v > b1) {
          b2 = b1;
          b1 = v;
        } else if (v > b2) {
          b2 = v;
        }
      }
      gscore = (sel_bias != nullptr && gs >= 2) ? b1 + b2 : b1;
    }
    int better = 0;
    for (int g = 0; g < n_groups; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g);
      better += (og > gscore || (og == gscore && g < lane)) ? 1 : 0;
    }
    const unsigned keep = __ballot_sync(0xffffffffu, lane < n_groups && better < groups_used);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (e < E && !((keep >> (e / gs)) & 1u)) sel[j] = -INFINITY;
    }
  }
  // iterative top-k: warp arg-max, ties to the lowest expert index
  int my_id[MOE_MAX_TOPK];
  float my_w[MOE_MAX_TOPK];
  float wsum = 0.f;
  for (int i = 0; i < k; ++i) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > bv || (sel[j] == bv && e < be)) {
        bv = sel[j];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    // owner lane publishes the unbiased score and retires the expert
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (lane + 32 * j == be) {
        w = score[j];
        sel[j] = -INFINITY;
      }
    }
    w = __shfl_sync(0xffffffffu, w, be & 31);
    my_id[i] = be;
    my_w[i] = w;
    wsum += w;
  }
  const float norm = (renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f) * weight_scale;
  // every lane holds the full list; lane (i mod 32) writes entry i
  for (int i = 0; i < k; ++i) {
    if (lane == (i & 31)) {
      ids[(size_t)t * k + i] = my_id[i];
      wts[(size_t)t * k + i] = my_w[i] * norm;
    }
  }
  if (scale != nullptr) {
    for (int el = lane; el < n_local; el += 32) {
      const int e = first_local + el;
      float s = 0.f;
      for (int i = 0; i < k; ++i) s += my_id[i] == e ? my_w[i] * norm : 0.f;
      scale[(size_t)el * scale_ld + t] = s;
    }
  }
}

// y [E, T, H] bf16 (expert-major), scale [E, scale_ld] f32, shared [T, H] bf16 or null -> out [T, H] bf16
static __global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ scale, int scale_ld,
                                   const __nv_bfloat16* __restrict__ shared, __nv_bfloat16* __restrict__ out, int E, int T,
                                   int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int H8 = H >> 3;
  for (int i = threadIdx.x; i < H8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (shared != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(shared + (size_t)t * H + i * 8);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int e = 0; e < E; ++e) {
      const float s = scale[(size_t)e * scale_ld + t];
      if (s == 0.f) continue;  // idle expert for this token: its rows were never written
      const uint4 v = *reinterpret_cast<const uint4*>(y + ((size_t)e * T + t) * H + i * 8);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]);
        acc[2 * j] += s * f.x;
        acc[2 * j + 1] += s * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + i * 8) = o;
  }
}

// ----------------------------------------------------------------------------- token dispatch (permute) for the grouped expert GEMM
// After routing, the rows that the experts held by THIS rank must process are gathered expert by expert into one
// contiguous matrix, so that the grouped GEMM multiplies every expert with exactly its own tokens (instead of all
// tokens with every active expert) and the whole layer stays on the device for any token count:
//   moe_permute_kernel   (ids [T, k]) -> offsets [n_local + 1], perm [T*k] (source token of gathered row r),
//                        inv [T, k] (gathered row that holds token t's k-th expert output, -1 if that expert
//                        lives on another rank)
//   moe_gather_kernel    Xg[r] = X[perm[r]]
//   grouped GEMMs        rows [offsets[e], offsets[e+1]) x expert e  (GroupArgs::row_offsets)
//   moe_combine_gathered out[t] = sum_k w[t, k] * Y[inv[t, k]] (+ shared expert)
// With expert parallelism the tokens are already on every rank (they leave the attention all-reduce replicated),
// so the dispatch crosses no link; what crosses NVLink is the combine, see moe_combine_exchange_kernel.
// One CTA: the lists of a step are a few thousand entries at most.
static __global__ void __launch_bounds__(1024)
moe_permute_kernel(const int* __restrict__ ids, int T, int k, int first_local, int n_local, int* __restrict__ offsets,
                   int* __restrict__ perm, int* __restrict__ inv) {
  __shared__ int cnt[MOE_MAX_EXPERTS];
  __shared__ int off[MOE_MAX_EXPERTS + 1];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int n = T * k;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i] - first_local;
    if (e >= 0 && e < n_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int e = 0; e < n_local; ++e) {
      off[e] = s;
      s += cnt[e];
    }
    off[n_local] = s;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= n_local; e += blockDim.x) offsets[e] = off[e];
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  // The order of the rows inside one expert's range depends on thread scheduling; nothing downstream depends on it
  // (every row is multiplied on its own, and the combine walks inv[] in the order of the routing list).
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i] - first_local;
    if (e >= 0 && e < n_local) {
      const int pos = off[e] + atomicAdd(&cnt[e], 1);
      perm[pos] = i / k;
      inv[i] = pos;
    } else {
      inv[i] = -1;
    }
  }
}

// Xg[r, :] = X[perm[r], :] for r < offsets[n_local]; 16-byte chunks, grid-stride over rows
static __global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ X, int H, const int* __restrict__ perm,
                                         const int* __restrict__ n_rows_dev, __nv_bfloat16* __restrict__ Xg) {
  pdl_launch_dependents();
  pdl_wait();
  const int R = *n_rows_dev;
  const int H8 = H >> 3;
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(X + (size_t)perm[r] * H);
    uint4* dst = reinterpret_cast<uint4*>(Xg + (size_t)r * H);
    for (int i = threadIdx.x; i < H8; i += blockDim.x) dst[i] = src[i];
  }
}

// SiLU(gate) * up over the first *n_rows_dev rows of a [rows, 2I] matrix
static __global__ void silu_mul_rows_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                            const int* __restrict__ n_rows_dev, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const int I8 = I >> 3;
  const size_t total = (size_t)(*n_rows_dev) * I8;
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
      os[j] = pack_bf16x2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = o;
  }
}

// weighted sum of one token's expert outputs for 8 columns starting at col
__device__ __forceinline__ void moe_combine8(const __nv_bfloat16* __restrict__ Y, int H, const int* __restrict__ inv,
                                             const float* __restrict__ wts, int k, int t, int col,
                                             const __nv_bfloat16* __restrict__ shared, float (&acc)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (shared != nullptr) {
    const uint4 v = *reinterpret_cast<const uint4*>(shared + (size_t)t * H + col);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]);
      acc[2 * j] = f.x;
      acc[2 * j + 1] = f.y;
    }
  }
  for (int i = 0; i < k; ++i) {  // in the order of the routing list: the same sum on every launch
    const int r = inv[(size_t)t * k + i];
    if (r < 0) continue;
    const float w = wts[(size_t)t * k + i];
    const uint4 v = *reinterpret_cast<const uint4*>(Y + (size_t)r * H + col);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]);
      acc[2 * j] += w * f.x;
      acc[2 * j + 1] += w * f.y;
    }
  }
}

// out[t] = sum_k w[t, k] * Y[inv[t, k]] (+ shared): the top-k weighted sum over the gathered expert outputs
static __global__ void moe_combine_gathered_kernel(const __nv_bfloat16* __restrict__ Y, const int* __restrict__ inv,
                                                   const float* __restrict__ wts, int k, const __nv_bfloat16* __restrict__ shared,
                                                   __nv_bfloat16* __restrict__ out, int T, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float acc[8];
    moe_combine8(Y, H, inv, wts, k, t, i * 8, shared, acc);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + i * 8) = ar_pack8(acc);
  }
}

// The same weighted sum fused with the all-reduce over the expert-parallel ranks: every CTA forms one
// [tg tokens x 128 columns] piece of this rank's partial combine in shared memory and hands it straight to the
// two-shot exchange over peer memory (ar_exchange), so the combine's result never goes to global memory before it
// crosses NVLink and there is no separate collective launch.  Grid = (H / 128 column tiles, token groups).
static __global__ void __launch_bounds__(128)
moe_combine_exchange_kernel(const ArArgs ar, const __nv_bfloat16* __restrict__ Y, const int* __restrict__ inv,
                            const float* __restrict__ wts, int k, const __nv_bfloat16* __restrict__ shared,
                            __nv_bfloat16* __restrict__ out, int T, int H, int tg) {
  extern __shared__ __align__(16) uint8_t cx_stage[];  // [tg][256] bytes
  __shared__ int s_call, s_abort;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * 128;
  const int t0 = blockIdx.y * tg;
  const int tmax = min(tg, T - t0);
  const int piece = blockIdx.y * gridDim.x + blockIdx.x;
  if (tid == 0) {
    s_call = ar.ctrl[0];
    s_abort = 0;
  }
  const int chunk = tid & 15, trow = tid >> 4;
  for (int t = trow; t < tmax; t += 8) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n0 + chunk * 8 < H) {
      float acc[8];
      moe_combine8(Y, H, inv, wts, k, t0 + t, n0 + chunk * 8, shared, acc);
      v = ar_pack8(acc);
    }
    *reinterpret_cast<uint4*>(cx_stage + t * 256 + chunk * 16) = v;
  }
  __syncthreads();
  ar_exchange(ar, cx_stage, s_call, piece, n0, t0, tmax, H, out, H, &s_abort, tid);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int done = atomicAdd(&ar.ctrl[1], 1);
    if (done == (int)(gridDim.x * gridDim.y) - 1) {
      ar.ctrl[1] = 0;
      __threadfence();
      ar.ctrl[0] = ar.ctrl[0] + 1;
    }
  }
}

}  // namespace oxb
