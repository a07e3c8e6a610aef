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

}  // namespace oxb
