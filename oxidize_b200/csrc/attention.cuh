// Paged GQA flash attention for decode, speculative verify and chunked prefill in one kernel.
//
// Work decomposition: a CTA owns (sequence, kv head, 16-row query tile, CTA split); a "row" is a
// (query token, head-in-group) pair, so the 8 query heads that share one KV head in the 70B / 8B
// shapes fill the M dimension of the tensor-core tile at decode time.  The CTA's four warps walk
// disjoint, strided sets of 16-token KV pages (one page = one MMA k-step), each with a private
// cp.async ring, and keep their own online-softmax state; partial (max, sum, O) results are
// merged in shared memory, and across CTA splits by whichever split finishes last (atomic ticket;
// split-KV with exact log-sum-exp merge, no second launch).  KV pages may be bf16, f16, or the symmetric per-32-channel q8 / q4
// encodings, which are decoded to bf16 on the way into shared memory.
//
// Covers what the reference does with flash_attn_decode(_splitk/_reduce)
// (oxidize-core/kernels/gemv_f32.cu:2035-2228), its CPU prefill attention
// (compute/flash_attention.rs:745) and the C port's block-table gather
// (oxidize-c/src/paged/paged_attention.c:751).
#pragma once
#include "common.cuh"

namespace oxb {

constexpr int ATT_WARPS = 4;
constexpr int ATT_PAGE = 16;
constexpr int ATT_STAGES = 3;

struct AttnArgs {
  const __nv_bfloat16* q;   // [T, nq, hd]
  __nv_bfloat16* out;       // [T, nq, hd]
  const void* kv_data;      // layer base
  const float* kv_scales;   // layer base (q8/q4) or null
  const int* block_tables;  // [B, max_blocks]
  const int* seq_lens;      // [B]
  const int* query_start;   // [B+1]
  int max_blocks, nq, nkv, kv_mode /*0 bf16,1 f16,2 q8,3 q4*/;
  int n_cta_splits, max_mtiles, window;
  int num_blocks;  // pages in the KV pool: block ids are checked against it
  float scale_log2;
  // soft-capped scores (Gemma-2): score = cap * tanh(q.k * scale / cap).  cap_log2 = cap * log2(e) (0 = off),
  // cap_arg = scale / cap
  float cap_log2, cap_arg;
  float* ws_o;   // [B*nkv*max_mtiles*n_cta_splits, 16, hd]
  float* ws_ml;  // [.., 16, 2]
  int* counters; // [B*nkv*max_mtiles] zero-initialised tickets (CTA splits only)
  unsigned long long* trace;  // optional: phase timestamps (globaltimer ns) of CTA (0,0,0), for latency analysis
};

#define ATT_STAMP(i)                                                                                          \
  do {                                                                                                        \
    if (a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {    \
      unsigned long long t_;                                                                                  \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                \
      a.trace[i] = t_;                                                                                        \
    }                                                                                                         \
  } while (0)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Bring one (K, V) page pair of a kv head into a warp-private stage with cp.async (one warp).
// bf16 / f16 pages land as 32 rows of HD 16-bit values with row stride HD*2+16 bytes (bank-
// conflict-free ldmatrix); q8 / q4 pages land raw: 32 rows of codes, then 32 rows of scales.
template <int HD>
__device__ __forceinline__ void load_page(uint8_t* stage, const AttnArgs& a, int blk, int kvh, int lane) {
  constexpr int ROWB = HD * 2 + 16;
  const size_t page_idx = ((size_t)blk * a.nkv + kvh) * 2;  // K page; V page follows
  if (a.kv_mode <= 1) {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.kv_data) + page_idx * ATT_PAGE * HD * 2;
    constexpr int CPR = HD * 2 / 16;  // 16-byte chunks per row
#pragma unroll
    for (int c = lane; c < 32 * CPR; c += 32) {
      const int row = c / CPR, col = c % CPR;
      cp_async16(stage + row * ROWB + col * 16, src + (size_t)c * 16);
    }
  } else {
    const int rowbytes = a.kv_mode == 2 ? HD : HD / 2;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.kv_data) + page_idx * ATT_PAGE * rowbytes;
    const uint8_t* sc = reinterpret_cast<const uint8_t*>(a.kv_scales + page_idx * ATT_PAGE * (HD / 32));
    const int ncode = 32 * rowbytes / 16;
    for (int c = lane; c < ncode; c += 32) cp_async16(stage + c * 16, src + (size_t)c * 16);
    constexpr int NSC = 32 * (HD / 32) * 4 / 16;
    for (int c = lane; c < NSC; c += 32) cp_async16(stage + 32 * rowbytes + c * 16, sc + (size_t)c * 16);
  }
}

// f16 pages: convert to bf16 in place.  q8 / q4 pages: decode codes * scale into `dec` (bf16,
// padded rows).  One warp; the caller synchronises the warp before the tensor-core reads.
template <int HD>
__device__ __forceinline__ void decode_page(uint8_t* stage, uint8_t* dec, int kv_mode, int lane) {
  constexpr int ROWB = HD * 2 + 16;
  if (kv_mode == 1) {
    for (int c = lane; c < 32 * HD / 2; c += 32) {
      const int row = c / (HD / 2), col = (c % (HD / 2)) * 2;
      uint32_t* p = reinterpret_cast<uint32_t*>(stage + row * ROWB + col * 2);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(p));
      *p = pack_bf16x2(f.x, f.y);
    }
  } else {
    const bool q8 = kv_mode == 2;
    const int rowbytes = q8 ? HD : HD / 2;
    const float* sc = reinterpret_cast<const float*>(stage + 32 * rowbytes);
    for (int c = lane; c < 32 * HD / 8; c += 32) {  // 8 channels per step
      const int row = c / (HD / 8), col = (c % (HD / 8)) * 8;
      const float s = sc[row * (HD / 32) + (col >> 5)];
      float v[8];
      if (q8) {
        const uint2 w = *reinterpret_cast<const uint2*>(stage + row * rowbytes + col);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[j] = ((float)((w.x >> (8 * j)) & 0xFF) - 127.f) * s;
          v[4 + j] = ((float)((w.y >> (8 * j)) & 0xFF) - 127.f) * s;
        }
      } else {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(stage + row * rowbytes + (col >> 1));
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ((float)((w >> (4 * j)) & 0xF) - 7.f) * s;
      }
      uint4 o;
      o.x = pack_bf16x2(v[0], v[1]);
      o.y = pack_bf16x2(v[2], v[3]);
      o.z = pack_bf16x2(v[4], v[5]);
      o.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(dec + row * ROWB + col * 2) = o;
    }
  }
}

// Merge the CTA-split partials of one (sequence, kv head, row tile): 128 threads = 16 rows x 8
// column segments.  Partials were written by other CTAs, so they are read through L2 (__ldcg).
template <int HD>
__device__ __forceinline__ void attn_merge_rows(const AttnArgs& a, int G, int b, int kvh, int mtile, int q0, int R, int tid) {
  const int row = tid >> 3, seg = (tid & 7) * (HD / 8);
  const int r = mtile * 16 + row;
  if (r >= R) return;
  const int gx = a.max_mtiles * a.n_cta_splits;
  const size_t task0 = ((size_t)b * a.nkv + kvh) * gx + (size_t)mtile * a.n_cta_splits;
  float M = -INFINITY;
  for (int s = 0; s < a.n_cta_splits; ++s) M = fmaxf(M, __ldcg(a.ws_ml + ((task0 + s) * 16 + row) * 2));
  float L = 0.f;
  float acc[HD / 8];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) acc[d] = 0.f;
  for (int s = 0; s < a.n_cta_splits; ++s) {
    const float ms = __ldcg(a.ws_ml + ((task0 + s) * 16 + row) * 2);
    const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
    L += w * __ldcg(a.ws_ml + ((task0 + s) * 16 + row) * 2 + 1);
    const float4* src = reinterpret_cast<const float4*>(a.ws_o + ((task0 + s) * 16 + row) * HD + seg);
#pragma unroll
    for (int d = 0; d < HD / 32; ++d) {
      const float4 v = __ldcg(src + d);
      acc[4 * d] += w * v.x;
      acc[4 * d + 1] += w * v.y;
      acc[4 * d + 2] += w * v.z;
      acc[4 * d + 3] += w * v.w;
    }
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  __nv_bfloat16* dst = a.out + ((size_t)(q0 + r / G) * a.nq + kvh * G + r % G) * HD + seg;
#pragma unroll
  for (int d = 0; d < HD / 8; d += 2) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16x2(acc[d] * inv, acc[d + 1] * inv);
}

template <int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_kernel(const AttnArgs a, int G /*q heads per kv head*/) {
  constexpr int ROWB = HD * 2 + 16;
  constexpr int STAGE_BYTES = 32 * ROWB;
  constexpr int KS = HD / 16;  // k-steps for QK^T
  constexpr int NT = HD / 8;   // n-tiles of the output
  extern __shared__ __align__(16) uint8_t att_smem[];
  ATT_STAMP(0);
  pdl_launch_dependents();
  // Everything up to the grid-dependency wait below reads only what earlier STEPS wrote: the step's
  // metadata (copied in before the first kernel) and KV pages that lie wholly below this step's rows.

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int mtile = blockIdx.x / a.n_cta_splits, csplit = blockIdx.x % a.n_cta_splits;
  const int q0 = a.query_start[b], qlen = a.query_start[b + 1] - q0;
  const int seq_len = a.seq_lens[b];
  const int R = qlen * G;
  const int row_base = mtile * 16;
  const size_t task = ((size_t)b * a.nkv + kvh) * gridDim.x + blockIdx.x;
  const bool active = row_base < R;

  // rows of this thread: r0 = row_base + g, r1 = r0 + 8
  int qtok[2], hg[2], qpos[2];
  bool rvalid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row_base + g + 8 * i;
    rvalid[i] = active && r < R;
    qtok[i] = rvalid[i] ? r / G : 0;
    hg[i] = rvalid[i] ? r % G : 0;
    qpos[i] = seq_len - qlen + qtok[i];
  }
  // last key position any row of the tile may see, first one (sliding window)
  int hi_pos = -1, lo_pos = 0;
  if (active) {
    const int last_row = min(R, row_base + 16) - 1;
    hi_pos = seq_len - qlen + last_row / G;
    if (a.window > 0) lo_pos = max(0, (seq_len - qlen + row_base / G) - a.window + 1);
  }
  const int page_lo = lo_pos / ATT_PAGE;
  const int n_pages = (active && hi_pos >= 0 && seq_len > 0) ? (hi_pos / ATT_PAGE + 1 - page_lo) : 0;
  const int stride = a.n_cta_splits * ATT_WARPS;
  const int first = csplit * ATT_WARPS + warp;  // this warp takes pages first, first+stride, ...
  const int my_pages = n_pages > first ? (n_pages - first + stride - 1) / stride : 0;

  float o[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  uint8_t* my_stage = att_smem + (size_t)warp * ATT_STAGES * STAGE_BYTES;
  const int* bt = a.block_tables + (size_t)b * a.max_blocks;
  // Page ids of this warp, fetched 32 at a time into registers (two batches held) so that the
  // block-table load never sits in front of a page load on the critical path.
  int id_base = 0;
  int ids_a = (lane < my_pages) ? bt[page_lo + first + lane * stride] : 0;
  int ids_b = (32 + lane < my_pages) ? bt[page_lo + first + (32 + lane) * stride] : 0;
  auto page_id = [&](int i) {
    const int r = i - id_base;
    const int va = __shfl_sync(0xffffffffu, ids_a, r & 31);
    const int vb = __shfl_sync(0xffffffffu, ids_b, r & 31);
    int id = r < 32 ? va : vb;
    if ((unsigned)id >= (unsigned)a.num_blocks) {  // never follow a bad block id: record it, read page 0
      if (lane == 0) oxb_report(OXB_BAD_BLOCK_ID, id);
      id = 0;
    }
    return id;
  };

  // (The KV pages are not requested into the L2 ahead of the dependency: behind an HBM-bound kernel such requests
  // compete with the stream that is still running.)
  pdl_wait();
  ATT_STAMP(1);
  // Q fragments (A operand), straight from global memory
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const __nv_bfloat16* qp = a.q + ((size_t)(q0 + qtok[i]) * a.nq + kvh * G + hg[i]) * HD + ks * 16 + 2 * t4;
      qf[ks][i] = rvalid[i] ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
      qf[ks][i + 2] = rvalid[i] ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
    }
  }

  ATT_STAMP(2);
  // prologue: fill the ring
#pragma unroll
  for (int s = 0; s < ATT_STAGES - 1; ++s) {
    if (s < my_pages) load_page<HD>(my_stage + s * STAGE_BYTES, a, page_id(s), kvh, lane);
    cp_async_commit();
  }

  for (int it = 0; it < my_pages; ++it) {
    if (it - id_base >= 32) {
      id_base += 32;
      ids_a = ids_b;
      ids_b = (id_base + 32 + lane < my_pages) ? bt[page_lo + first + (id_base + 32 + lane) * stride] : 0;
    }
    const int nxt = it + ATT_STAGES - 1;
    if (nxt < my_pages) load_page<HD>(my_stage + (nxt % ATT_STAGES) * STAGE_BYTES, a, page_id(nxt), kvh, lane);
    cp_async_commit();
    cp_async_wait<ATT_STAGES - 1>();
    __syncwarp();
    if (it == 0) ATT_STAMP(3);
    uint8_t* st = my_stage + (it % ATT_STAGES) * STAGE_BYTES;
    if (a.kv_mode != 0) {
      uint8_t* dec = att_smem + (size_t)(ATT_WARPS * ATT_STAGES + warp) * STAGE_BYTES;
      decode_page<HD>(st, dec, a.kv_mode, lane);
      if (a.kv_mode >= 2) st = dec;
      __syncwarp();
    }
    const uint32_t k_base = smem_u32(st), v_base = k_base + 16 * ROWB;
    const int page = page_lo + first + it * stride;

    // S = Q K^T for 16 tokens: 2 n-tiles
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t addr0 = k_base + ((mi >> 1) * 8 + r) * ROWB + (mi & 1) * 16;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(addr0 + ks * 32, b0, b1, b2, b3);
        mma_bf16_16816(s[0], qf[ks], b0, b1);
        mma_bf16_16816(s[1], qf[ks], b2, b3);
      }
    }
    // scale, mask, online softmax (rows g and g+8; a quad holds one row's 16 scores)
    const int key0 = page * ATT_PAGE;
    float p[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + nt * 8 + 2 * t4 + e;
          float v = a.cap_log2 > 0.f ? a.cap_log2 * tanhf(s[nt][2 * i + e] * a.cap_arg) : s[nt][2 * i + e] * a.scale_log2;
          const bool ok = rvalid[i] && key <= qpos[i] && (a.window <= 0 || key > qpos[i] - a.window);
          v = ok ? v : -INFINITY;
          s[nt][2 * i + e] = v;
          mx = fmaxf(mx, v);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[i], mx);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m_run[i] - base);  // 0 when m_run was -inf
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s[nt][2 * i + e] - base);
          p[nt][2 * i + e] = pv;
          sum += pv;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[i] = l_run[i] * corr + sum;
      m_run[i] = m_new;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        o[nt][2 * i] *= corr;
        o[nt][2 * i + 1] *= corr;
      }
    }
    // O += P V : P (16x16) as A fragment, V page as B via transposing ldmatrix
    uint32_t pf[4];
    pf[0] = pack_bf16x2(p[0][0], p[0][1]);
    pf[1] = pack_bf16x2(p[0][2], p[0][3]);
    pf[2] = pack_bf16x2(p[1][0], p[1][1]);
    pf[3] = pack_bf16x2(p[1][2], p[1][3]);
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t addr0 = v_base + ((mi & 1) * 8 + r) * ROWB + (mi >> 1) * 16;
#pragma unroll
      for (int nt = 0; nt < NT; nt += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(addr0 + nt * 16, b0, b1, b2, b3);
        mma_bf16_16816(o[nt], pf, b0, b1);
        mma_bf16_16816(o[nt + 1], pf, b2, b3);
      }
    }
    __syncwarp();
  }
  ATT_STAMP(4);
  cp_async_wait<0>();
  __syncthreads();
  ATT_STAMP(5);

  // ---- merge the four warps through shared memory (reusing the stage area)
  float* mo = reinterpret_cast<float*>(att_smem);             // [4][16][HD]
  float* mml = mo + ATT_WARPS * 16 * HD;                       // [4][16][2]
  // (rows past R do not exist — at decode with 8 query heads per KV head that is half of the tile: they are
  // neither staged nor merged)
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (rvalid[i]) {
        float2* dst = reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + g + 8 * i) * HD + nt * 8 + 2 * t4);
        *dst = make_float2(o[nt][2 * i], o[nt][2 * i + 1]);
      }
    }
  }
  if (t4 == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (rvalid[i]) {
        mml[(warp * 16 + g + 8 * i) * 2] = m_run[i];
        mml[(warp * 16 + g + 8 * i) * 2 + 1] = l_run[i];
      }
    }
  }
  __syncthreads();
  {
    const int row = threadIdx.x >> 3;          // 0..15
    const int seg = (threadIdx.x & 7) * (HD / 8);
    const int r = row_base + row;
    const bool valid = active && r < R;
    float M = -INFINITY;
    float L = 0.f, wgt[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) wgt[w] = 0.f;
    if (valid) {
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, mml[(w * 16 + row) * 2]);
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) {
        const float mw = mml[(w * 16 + row) * 2];
        wgt[w] = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L += wgt[w] * mml[(w * 16 + row) * 2 + 1];
      }
    }
    if (a.n_cta_splits == 1) {
      if (valid) {
        const float inv = L > 0.f ? 1.f / L : 0.f;
        __nv_bfloat16* dst = a.out + ((size_t)(q0 + r / G) * a.nq + kvh * G + r % G) * HD + seg;
        for (int d = 0; d < HD / 8; d += 2) {
          float v0 = 0.f, v1 = 0.f;
#pragma unroll
          for (int w = 0; w < ATT_WARPS; ++w) {
            v0 += wgt[w] * mo[((size_t)w * 16 + row) * HD + seg + d];
            v1 += wgt[w] * mo[((size_t)w * 16 + row) * HD + seg + d + 1];
          }
          *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16x2(v0 * inv, v1 * inv);
        }
      }
    } else {
      if (valid) {
        float4* wo = reinterpret_cast<float4*>(a.ws_o + (task * 16 + row) * HD + seg);
        for (int d = 0; d < HD / 8; d += 4) {
          float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int w = 0; w < ATT_WARPS; ++w) {
            const float4 x = *reinterpret_cast<const float4*>(mo + ((size_t)w * 16 + row) * HD + seg + d);
            v[0] += wgt[w] * x.x;
            v[1] += wgt[w] * x.y;
            v[2] += wgt[w] * x.z;
            v[3] += wgt[w] * x.w;
          }
          wo[d >> 2] = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
      if ((threadIdx.x & 7) == 0) {
        a.ws_ml[(task * 16 + row) * 2] = valid ? M : -INFINITY;
        a.ws_ml[(task * 16 + row) * 2 + 1] = valid ? L : 0.f;
      }
    }
  }
  ATT_STAMP(6);
  if (a.n_cta_splits > 1) {
    // the last CTA split of this row tile to finish merges all partials (no second launch)
    __shared__ int s_ticket;
    __threadfence();
    __syncthreads();
    int* cnt = a.counters + ((size_t)b * a.nkv + kvh) * a.max_mtiles + mtile;
    if (threadIdx.x == 0) s_ticket = atomicAdd(cnt, 1);
    __syncthreads();
    if (s_ticket == a.n_cta_splits - 1) {
      __threadfence();
      attn_merge_rows<HD>(a, G, b, kvh, mtile, q0, R, threadIdx.x);
      if (threadIdx.x == 0) *cnt = 0;  // re-armed for the next launch / graph replay
    }
  }
  ATT_STAMP(7);
}

}  // namespace oxb
