// Device sampling: one CTA per logits row.
//
// Row r draws with temperature[r] (<= 0: greedy with the configured tie rule), top_k[r] (0: off),
// top_p[r], min_p[r] and the host-supplied uniform random[r], in the order of the reference's
// sampler (oxidize-core/src/model/sampling.rs:268-463): softmax over the full vocabulary, keep a
// prefix of the descending order (top-k, then top-p "through the first index whose cumulative
// mass reaches p", then min-p), inverse CDF with target = random * sum(kept).  Rows without any
// filter use the reference's single-pass rule: inverse CDF in *index* order (:465-490).
//
// The kept prefix is found without sorting the vocabulary: tokens are ordered by a 64-bit key
// (probability bits descending, index ascending) and every question about the sorted order
// ("how many tokens / how much mass lies before key x") is answered by a radix descent over
// the key bits — 8 bits per pass, per-bin counts and masses accumulated in shared memory.
#pragma once
#include "common.cuh"

namespace oxb {

constexpr int SMP_THREADS = 1024;

struct BlockScan {
  // inclusive scan of one float per thread across the block; returns (inclusive, block total)
  __device__ static float2 run(float v, float* warp_tot /*[32]*/) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = x;
    __syncthreads();
    float base = 0.f, total = 0.f;
    for (int w = 0; w < nw; ++w) {
      const float t = warp_tot[w];
      if (w < warp) base += t;
      total += t;
    }
    return make_float2(x + base, total);
  }
};

// f(i, row[i]) for every i < V, the block's threads striding over the row.  Rows that start on a 16-byte boundary are
// read as float4 with four loads in flight per thread: a pass is a stream of the row out of the L2, and one scalar
// load per iteration leaves every thread waiting out a full memory latency per element.
template <class F>
__device__ __forceinline__ void row_for_each(const float* __restrict__ row, int V, F f) {
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
#pragma unroll 4
    for (int q = threadIdx.x; q < n4; q += blockDim.x) {
      const float4 v = r4[q];
      f(4 * q, v.x);
      f(4 * q + 1, v.y);
      f(4 * q + 2, v.z);
      f(4 * q + 3, v.w);
    }
    for (int i = (n4 << 2) + threadIdx.x; i < V; i += blockDim.x) f(i, row[i]);
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < V; i += blockDim.x) f(i, row[i]);
  }
}

// First index (in index order) at which the running total of weight(i) exceeds `target`, or 0x7fffffff.  Every thread
// sums a contiguous slice of the row, ONE block scan orders the slices, and the thread whose slice holds the crossing
// walks it again: two passes over the row and three block barriers, whatever the vocabulary size (a scan per 1024
// elements costs 125 scans for a 128 k vocabulary).  *s_out must hold 0x7fffffff on entry (set before a barrier).
template <class Weight>
__device__ __forceinline__ int locate_in_index_order(const float* __restrict__ row, int V, float target, Weight weight,
                                                     float* red, int* s_out) {
  const int per = (((V + (int)blockDim.x - 1) / (int)blockDim.x) + 3) & ~3;  // slices start on multiples of four
  const int b = min((int)threadIdx.x * per, V), e = min(b + per, V);
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  auto slice = [&](auto&& g) {  // g(i, row[i]) over this thread's slice, in index order
    int i = b;
    if (vec) {
#pragma unroll 2
      for (; i + 4 <= e; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        if (!g(i, v.x) || !g(i + 1, v.y) || !g(i + 2, v.z) || !g(i + 3, v.w)) return;
      }
    }
    for (; i < e; ++i)
      if (!g(i, row[i])) return;
  };
  float local = 0.f;
  slice([&](int i, float v) {
    local += weight(i, v);
    return true;
  });
  const float2 sc = BlockScan::run(local, red);
  const float before = sc.x - local;
  if (local > 0.f && sc.x > target && before <= target) {
    float run = before;
    slice([&](int i, float v) {
      const float w = weight(i, v);
      if (w > 0.f && run + w > target) {
        atomicMin(s_out, i);
        return false;
      }
      run += w;
      return true;
    });
  }
  __syncthreads();
  return *s_out;
}

// monotone map float -> uint32 (larger float -> larger uint); probabilities are >= 0
__device__ __forceinline__ uint32_t prob_bits(float p) { return __float_as_uint(p); }

// For the tokens whose probability bits match `prefix` on the top `done_bits` bits, accumulate
// per-bin (next 8 bits) count and mass into shared histograms.
__device__ __forceinline__ void radix_pass(const float* __restrict__ row, int V, float mx, float inv_t, uint32_t prefix,
                                           int done_bits, int* cnt, float* mass, int* wcnt, float* wmass) {
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    cnt[i] = 0;
    mass[i] = 0.f;
  }
  if (done_bits == 0 && wcnt[32 * 64] != 0) {
    // the first-pass histogram of this row was built by an earlier descent: reuse it
    __syncthreads();
    if (threadIdx.x < 64) {
      cnt[threadIdx.x] = wcnt[32 * 64 + 1 + threadIdx.x];
      mass[threadIdx.x] = wmass[32 * 64 + 1 + threadIdx.x];
    }
    __syncthreads();
    return;
  }
  if (done_bits == 0) {
    // First pass: EVERY token lands in one of a handful of bins (probabilities are <= 1, so the top
    // byte of their bits is <= 63, and real rows use ~10 of those), and 1024 threads adding into the
    // same few shared-memory words serialise.  Each warp therefore fills a private 64-bin histogram,
    // summed afterwards (this pass was 95 % of the kernel's time before).
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 32 * 64; i += blockDim.x) {
      wcnt[i] = 0;
      wmass[i] = 0.f;
    }
    __syncthreads();
    row_for_each(row, V, [&](int, float v) {
      const float p = __expf((v - mx) * inv_t);
      const int bin = min((int)(prob_bits(p) >> 24), 63);
      atomicAdd(&wcnt[warp * 64 + bin], 1);
      atomicAdd(&wmass[warp * 64 + bin], p);
    });
    __syncthreads();
    if (threadIdx.x < 64) {
      int c = 0;
      float m = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
        c += wcnt[w * 64 + threadIdx.x];
        m += wmass[w * 64 + threadIdx.x];
      }
      cnt[threadIdx.x] = c;
      mass[threadIdx.x] = m;
      wcnt[32 * 64 + 1 + threadIdx.x] = c;  // kept for the row's next descent
      wmass[32 * 64 + 1 + threadIdx.x] = m;
    }
    if (threadIdx.x == 0) wcnt[32 * 64] = 1;
    __syncthreads();
    return;
  }
  __syncthreads();
  const int shift = 24 - done_bits;
  row_for_each(row, V, [&](int, float v) {
    const float p = __expf((v - mx) * inv_t);
    const uint32_t b = prob_bits(p);
    if ((b >> (32 - done_bits)) == (prefix >> (32 - done_bits))) {
      const int bin = (b >> shift) & 0xFF;
      atomicAdd(&cnt[bin], 1);
      atomicAdd(&mass[bin], p);
    }
  });
  __syncthreads();
}

// Find the probability-bits value x such that, walking the vocabulary in descending probability,
// the walk crosses the boundary defined by (count limit, mass limit) inside the tokens whose
// bits equal x.  Returns x and the count / mass strictly above x.
__device__ void radix_descend(const float* row, int V, float mx, float inv_t, int count_limit, float mass_limit,
                              int* cnt, float* mass, int* wcnt, float* wmass, int* s_i, float* s_f, uint32_t& x, int& cnt_above,
                              float& mass_above) {
  uint32_t prefix = 0;
  int ca = 0;
  float ma = 0.f;
  for (int done = 0; done < 32; done += 8) {
    radix_pass(row, V, mx, inv_t, prefix, done, cnt, mass, wcnt, wmass);
    if (threadIdx.x < 32) {
      // Walk the 256 bins from the top until the boundary falls inside one; bin 0 ends the walk in any case.  One
      // warp does it: lane l sums bins 255 - 8l .. 248 - 8l, a shuffle scan gives every lane the totals above its
      // bins, each lane then looks for the crossing among its own eight, and the lowest lane that finds one wins.
      const int lane = threadIdx.x;
      int lc = 0;
      float lm = 0.f;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        lc += cnt[255 - (lane * 8 + t)];
        lm += mass[255 - (lane * 8 + t)];
      }
      int pc = lc;
      float pm = lm;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int yc = __shfl_up_sync(0xffffffffu, pc, o);
        const float ym = __shfl_up_sync(0xffffffffu, pm, o);
        if (lane >= o) {
          pc += yc;
          pm += ym;
        }
      }
      int c = ca + pc - lc;
      float m = ma + pm - lm;
      int found = -1;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int bin = 255 - (lane * 8 + t);
        if (found < 0) {
          if (bin == 0 || c + cnt[bin] >= count_limit || m + mass[bin] >= mass_limit) {
            found = bin;
          } else {
            c += cnt[bin];
            m += mass[bin];
          }
        }
      }
      const unsigned hit = __ballot_sync(0xffffffffu, found >= 0);
      if (lane == __ffs(hit) - 1) {
        s_i[0] = found;
        s_i[1] = c;
        s_f[0] = m;
      }
    }
    __syncthreads();
    prefix |= (uint32_t)s_i[0] << (24 - done);
    ca = s_i[1];
    ma = s_f[0];
    __syncthreads();
  }
  x = prefix;
  cnt_above = ca;
  mass_above = ma;
}

static __global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ random, int tie_highest, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ int cnt[256];
  __shared__ float mass[256];
  __shared__ int wcnt[32 * 64 + 65];     // per-warp histograms of the first radix pass; [2048] = "saved" flag,
  __shared__ float wmass[32 * 64 + 65];  // [2049..2112] = the summed first-pass histogram, reused by the draw
  __shared__ int s_i[4];
  __shared__ float s_f[4];
  __shared__ int s_best;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) wcnt[32 * 64] = 0;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float T = temperature[r];
  // ---- max (and greedy argmax)
  float mx = -INFINITY;
  int bi = -1;
  row_for_each(row, V, [&](int i, float v) {
    // a thread visits its indices in increasing order, so "later wins ties" is the highest-index rule
    if (bi < 0 || v > mx || (v == mx && tie_highest)) {
      if (!(v != v)) {
        mx = v;
        bi = i;
      }
    }
  });
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float sv[32];
    __shared__ int si[32];
    auto better = [&](float v, int i, float bv, int b) {
      if (i < 0) return false;
      if (b < 0) return true;
      return v > bv || (v == bv && (tie_highest ? i > b : i < b));
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, mx, bi)) {
        mx = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      sv[warp] = mx;
      si[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
      mx = sv[lane];
      bi = si[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, mx, bi)) {
          mx = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        s_f[1] = mx;
        s_best = bi < 0 ? 0 : bi;
      }
    }
    __syncthreads();
    mx = s_f[1];
  }
  const int k = top_k[r];
  if (T <= 0.f || k == 1 || !(mx > -INFINITY)) {
    if (threadIdx.x == 0) out[r] = s_best;
    return;
  }
  const float inv_t = 1.f / T;
  // ---- total mass
  float part = 0.f;
  row_for_each(row, V, [&](int, float v) { part += __expf((v - mx) * inv_t); });
  const float total = block_sum(part, red);
  if (!(total > 0.f) || !isfinite(total)) {
    if (threadIdx.x == 0) out[r] = s_best;
    return;
  }
  const float tp = top_p[r], mp = min_p[r], rnd = random[r];
  const bool filtered = k > 0 || tp < 1.f || mp > 0.f;
  if (threadIdx.x == 0) s_i[2] = 0x7fffffff;
  __syncthreads();
  if (!filtered) {
    // inverse CDF in index order
    const float target = rnd * total;
    const int tok = locate_in_index_order(row, V, target, [&](int, float v) { return __expf((v - mx) * inv_t); }, red, &s_i[2]);
    if (threadIdx.x == 0) out[r] = tok == 0x7fffffff ? V - 1 : tok;
    return;
  }
  // ---- filtered: find the end of the kept prefix of the descending order
  // kept = first min(top_k, n_p, n_minp) tokens, where n_p counts tokens whose mass-before < top_p * total
  const int klim = k > 0 ? k : V;
  const float plim = tp < 1.f ? tp * total : INFINITY;
  uint32_t xb;
  int c_above;
  float m_above;
  radix_descend(row, V, mx, inv_t, klim, plim, cnt, mass, wcnt, wmass, s_i, s_f, xb, c_above, m_above);
  // tokens with bits > xb are kept entirely; tokens with bits == xb are kept in index order while
  // the limits allow; min-p cuts by value on top of that
  const float pmin_keep = mp > 0.f ? mp * 1.0f /* p_max = exp(0) = 1 */ : 0.f;
  // kept mass: (a) everything above xb that also passes min-p, (b) the admitted part of the tie group
  // First count how many of the tie group are admitted.
  const float px = __uint_as_float(xb);
  int admit = 0;
  {
    int room_k = klim - c_above;
    // through the first index whose cumulative reaches top_p: tokens whose mass-before < plim
    float room_p = plim - m_above;
    int by_p = px > 0.f ? (int)ceilf(room_p / px) : 0x7fffffff;
    if (room_p == INFINITY) by_p = 0x7fffffff;
    admit = max(0, min(room_k, by_p));
    if (c_above == 0 && admit == 0) admit = 1;  // always keep the top token
  }
  // kept sum and size of the tie group, one pass
  float ks = 0.f;
  int tc = 0;
  row_for_each(row, V, [&](int, float v) {
    const float p = __expf((v - mx) * inv_t);
    const uint32_t pb = prob_bits(p);
    if (pb > xb && p >= pmin_keep) ks += p;
    tc += pb == xb;
  });
  float kept = block_sum(ks, red);
  const int tie_total = (int)(block_sum((float)tc, red) + 0.5f);
  const bool ties_pass_minp = px >= pmin_keep;
  const int tie_kept = ties_pass_minp ? min(admit, tie_total) : 0;
  kept += (float)tie_kept * px;
  if (!(kept > 0.f)) {
    if (threadIdx.x == 0) out[r] = s_best;
    return;
  }
  // ---- draw: walk the kept prefix in sorted order until the running mass exceeds target
  const float target = rnd * kept;
  uint32_t yb;
  int c2;
  float m2;
  // boundary where mass-before exceeds target (no count limit); restrict to kept tokens by
  // noting that kept tokens form a prefix, so the walk never leaves it when target < kept
  radix_descend(row, V, mx, inv_t, 0x7fffffff, nextafterf(target, INFINITY), cnt, mass, wcnt, wmass, s_i, s_f, yb, c2, m2);
  // inside the tie group of yb, tokens are ordered by index: pick the j-th
  const float py = __uint_as_float(yb);
  int j = py > 0.f ? (int)floorf((target - m2) / py) : 0;
  if (yb == xb) j = min(j, max(tie_kept - 1, 0));
  j = max(j, 0);
  // select the j-th token (by index) with bits == yb
  if (threadIdx.x == 0) s_i[2] = 0x7fffffff;
  __syncthreads();
  locate_in_index_order(row, V, (float)j + 0.5f,
                        [&](int, float v) { return prob_bits(__expf((v - mx) * inv_t)) == yb ? 1.f : 0.f; }, red, &s_i[2]);
  if (threadIdx.x == 0) {
    int tok = s_i[2];
    if (tok == 0x7fffffff) tok = s_best;  // numerical corner: fall back to the mode
    out[r] = tok;
  }
}

// ----------------------------------------------------------------------------- speculative verification
// One CTA per sequence walks its K drafted tokens against the K+1 rows of target logits that one batched forward
// produced.  Greedy sequences (temperature <= 0) keep drafts while they equal the target's argmax.  Sampled
// sequences use the rejection rule that leaves the output distributed exactly as the target's:
//   accept draft d_i with probability min(1, p_i(d_i) / q_i(d_i));
//   at the first rejection emit a token drawn from normalise(max(p_i - q_i, 0)) and stop;
//   if all K were accepted emit a bonus token drawn from p_K.
// p_i = softmax(target row i / T), q_i = softmax(draft row i / T).  Each decision consumes uniforms handed in by
// the host: u[2i] for the accept test, u[2i + 1] for the draw, u[2K] for the bonus token.  Draws are inverse-CDF
// in index order over a block-wide scan, so a given set of uniforms gives one result on any launch.
// Acceptance rule and bonus token of the reference: speculative_accept (oxidize-core/src/model/sampling.rs:492-623).
struct SpecVerifyArgs {
  const float* target;       // [rows, V] target logits, row stride ld_t
  const float* draft;        // [S * K, V] draft logits, row stride ld_d (row s * K + i); may be null for greedy-only
  const int* draft_tokens;   // [S, K]
  const int* row0;           // [S] first target row of each sequence
  const int* n_draft;        // [S] drafts of each sequence (<= K)
  const float* temperature;  // [S]
  const float* uniforms;     // [S, 2K + 1]
  int* out_tokens;           // [S, K + 1]
  int* out_count;            // [S] tokens emitted (accepted drafts + 1)
  int V, K, ld_t, ld_d, tie_highest;
};

// block-wide (max, argmax) and sum helpers over a logits row
__device__ __forceinline__ void spec_row_max(const float* row, int V, int tie_highest, float* sv, int* si, float& mx, int& arg) {
  float best = -INFINITY;
  int bi = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v == v && (bi < 0 || v > best || (v == best && tie_highest))) {
      best = v;
      bi = i;
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
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  best = sv[0];
  bi = si[0];
  for (int w = 1; w < nw; ++w)
    if (better(sv[w], si[w], best, bi)) {
      best = sv[w];
      bi = si[w];
    }
  mx = best;
  arg = bi < 0 ? 0 : bi;
}

__device__ __forceinline__ float spec_block_sum(float v, float* sv) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sv[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += sv[w];
  return t;
}

// Draw from the unnormalised weights w(i) >= 0, i in [0, V), by inverse CDF in index order: each thread owns a
// contiguous chunk.  `wf(i)` evaluates the weight.  Returns the index (all threads get it).
template <class WF>
__device__ __forceinline__ int spec_draw(int V, float u, WF wf, float* sv, int* s_pick, int fallback) {
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int b = threadIdx.x * per, e = min(V, b + per);
  float local = 0.f;
  for (int i = b; i < e; ++i) local += wf(i);
  const float2 sc = BlockScan::run(local, sv);
  const float total = sc.y;
  if (threadIdx.x == 0) *s_pick = -1;
  __syncthreads();
  if (total > 0.f && total == total) {
    const float target = u * total;
    const float before = sc.x - local;
    // the thread whose chunk contains the target (the last chunk takes what rounding leaves over)
    const bool mine = local > 0.f && target >= before && (target < sc.x || sc.x >= total);
    if (mine) {
      float c = before;
      int pick = -1;
      for (int i = b; i < e; ++i) {
        const float w = wf(i);
        if (w > 0.f) {
          pick = i;
          c += w;
          if (c > target) break;
        }
      }
      if (pick >= 0) atomicMax(s_pick, pick);
    }
  }
  __syncthreads();
  const int r = *s_pick;
  __syncthreads();
  return r >= 0 ? r : fallback;
}

static __global__ void __launch_bounds__(SMP_THREADS)
spec_verify_kernel(const SpecVerifyArgs a) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_pick;
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x;
  const int K = a.K, nd = min(a.n_draft[s], K);
  const float T = a.temperature[s];
  const float* u = a.uniforms + (size_t)s * (2 * K + 1);
  int* out = a.out_tokens + (size_t)s * (K + 1);
  int n_out = 0;
  bool stopped = false;
  for (int i = 0; i <= nd && !stopped; ++i) {
    const float* trow = a.target + (size_t)(a.row0[s] + i) * a.ld_t;
    float tmax;
    int targ;
    spec_row_max(trow, a.V, a.tie_highest, sv, si, tmax, targ);
    if (T <= 0.f || a.draft == nullptr) {
      // greedy: the target's argmax decides; a draft is kept only if it is that token
      if (threadIdx.x == 0) out[n_out] = targ;
      ++n_out;
      stopped = i == nd || a.draft_tokens[(size_t)s * K + i] != targ;
      continue;
    }
    const float inv_t = 1.f / T;
    float zp = 0.f;
    for (int v = threadIdx.x; v < a.V; v += blockDim.x) zp += __expf((trow[v] - tmax) * inv_t);
    zp = spec_block_sum(zp, sv);
    const float inv_zp = 1.f / zp;
    if (i == nd) {
      // every draft was accepted: bonus token from the target's own distribution
      const int tok = spec_draw(a.V, u[2 * K], [&](int v) { return __expf((trow[v] - tmax) * inv_t); }, sv, &s_pick, targ);
      if (threadIdx.x == 0) out[n_out] = tok;
      ++n_out;
      break;
    }
    const float* drow = a.draft + (size_t)(s * K + i) * a.ld_d;
    float dmax;
    int darg;
    spec_row_max(drow, a.V, a.tie_highest, sv, si, dmax, darg);
    float zq = 0.f;
    for (int v = threadIdx.x; v < a.V; v += blockDim.x) zq += __expf((drow[v] - dmax) * inv_t);
    zq = spec_block_sum(zq, sv);
    const float inv_zq = 1.f / zq;
    const int d = a.draft_tokens[(size_t)s * K + i];
    const float pd = __expf((trow[d] - tmax) * inv_t) * inv_zp;
    const float qd = __expf((drow[d] - dmax) * inv_t) * inv_zq;
    const float ratio = qd > 0.f ? pd / qd : 1.f;
    if (u[2 * i] < fminf(1.f, ratio)) {
      if (threadIdx.x == 0) out[n_out] = d;
      ++n_out;
      continue;
    }
    // rejected: draw from the part of the target's mass that the draft does not cover
    const int tok = spec_draw(
        a.V, u[2 * i + 1],
        [&](int v) { return fmaxf(__expf((trow[v] - tmax) * inv_t) * inv_zp - __expf((drow[v] - dmax) * inv_t) * inv_zq, 0.f); }, sv,
        &s_pick, targ);
    if (threadIdx.x == 0) out[n_out] = tok;
    ++n_out;
    stopped = true;
  }
  if (threadIdx.x == 0) a.out_count[s] = n_out;
}

}  // namespace oxb
