// Y[T, N] = X[T, K] · W[N, K]^T  (bf16 in, fp32 accumulate in TMEM, bf16 out) for sm_100a.
//
// Weight-stationary orientation: the UMMA M dimension (128) runs over weight rows, the UMMA N
// dimension (TN = 16..256) over tokens, so a decode batch of 1..256 tokens is ONE instruction
// shape and the kernel is a pure weight stream: every CTA pulls 128-row × 64-column weight
// tiles with TMA (128-byte swizzle) through a deep mbarrier ring, one elected thread issues
// tcgen05.mma into a TMEM accumulator, and four epilogue warps read it back with tcgen05.ld.
// Small-N projections are split along K across CTAs so that all 148 SMs stream; the CTAs of a
// tile meet at an arrive counter and each reduces its own slice of the tile's tokens from the
// fp32 partials in a fixed split order, which keeps the result bit-reproducible.
//
// Replaces the reference's cuBLAS SGEMM / cuBLASLt f16 prefill GEMMs and its f16 GEMV
// (oxidize-core/src/backends/cuda/gemm.rs:100, oxidize-cpp/src/cuda/gemm.cu:43,141-201).
#pragma once
#include "common.cuh"
#include "comm_fused.cuh"
#include "mmq_producer.cuh"

namespace oxb {

constexpr int GEMM_BM = 128;  // weight rows per tile (UMMA M)
constexpr int GEMM_BK = 64;   // bf16 per k-block = one 128-byte swizzle row
// Warp roles.  Warps 0-3: epilogue (TMEM lane quarter = warp % 4).  Warp 4: TMA.  Warp 5: MMA issuer (owns the TMEM
// allocation).  Packed weights add warps 6-7 (idle: they complete the second warpgroup, so that register budgets can be
// moved between whole warpgroups) and, from warp 8 on, the dequant producers.
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_WARP_TMA = 4, GEMM_WARP_MMA = 5, GEMM_WARP_PRODUCER0 = 8;
#ifndef OXB_MMQ_GROUPS
#define OXB_MMQ_GROUPS 4
#endif
constexpr int MMQ_GROUPS = OXB_MMQ_GROUPS;  // producer groups of four warps (one weight row per thread); group g decodes k-blocks g, g + MMQ_GROUPS, ...
constexpr int GEMM_THREADS_MMQ = 32 * GEMM_WARP_PRODUCER0 + 128 * MMQ_GROUPS;
// Register budgets of the packed-weight kernel (setmaxnreg): registers per thread at launch, then per warpgroup role.
// A CTA can only redistribute what it was launched with, so the budgets must add up to exactly that.
constexpr int MMQ_REGS_LAUNCH = 80, MMQ_REGS_EPILOGUE = 184, MMQ_REGS_CONTROL = 40, MMQ_REGS_PRODUCER = 64;
static_assert(128 * MMQ_REGS_EPILOGUE + 128 * MMQ_REGS_CONTROL + 128 * MMQ_GROUPS * MMQ_REGS_PRODUCER ==
                  GEMM_THREADS_MMQ * MMQ_REGS_LAUNCH,
              "warpgroup register budgets must add up to the launch allocation");
static_assert(GEMM_THREADS_MMQ * (MMQ_REGS_LAUNCH + 8) > 65536, "launch bounds must pin the kernel to MMQ_REGS_LAUNCH registers");


// k-blocks (16 KB of weights each) a CTA requests into the L2 before the grid dependency resolves
// (GroupArgs::l2_prefetch_kb, set per launch).  Behind an HBM-bound kernel this LOSES 10-20% (the
// requests compete with the running kernel's own stream), so the default is 0; behind a collective,
// whose wait leaves HBM idle, it turns the wait into the next GEMM's weight stream.
extern int g_oxb_gemm_l2_prefetch_kb;

template <int TN>
struct GemmTile {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = TN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Decode-sized tiles keep the ring below half of the SM's shared memory: two CTAs fit per SM, so
  // the CTAs of the NEXT kernel in the stream (launched early by programmatic dependent launch) can
  // already stream their weights while this kernel drains, and a split-K grid may hold 2 CTAs per SM.
  static constexpr int STAGES = TN <= 16 ? 6 : TN == 32 ? 5 : TN == 64 ? 4 : (TN == 128 ? 6 : 4);
  static constexpr int CTAS_PER_SM = TN <= 64 ? 2 : 1;
  // One accumulator per tile.  (Spreading the four k-steps of a k-block over separate accumulators, to break the
  // dependency chain of back-to-back MMAs, changed nothing measurable.)
  static constexpr int ACC_COLS = TN < 32 ? 32 : TN;  // TMEM columns of the accumulator
  static constexpr int TMEM_COLS = ACC_COLS;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ + 1024 /*token scales*/;
};

// Packed weights with decode-sized token tiles are staged through shared memory: one TMA box of
// 128 rows x one 256-value super-block of every row of the tile per four k-blocks, in a ring of RING boxes
// (one being decoded, the others in flight: a box is small against the latency of its fetch, so the
// ring, not the decoders, sets how many bytes the SM keeps in flight); the producer warps decode from there.  (Reading the packed rows straight from global memory, one thread per
// row, makes every warp-wide load touch 32 cache lines.)  A Q6_K super-block is 210 bytes, which TMA cannot
// address (16-byte rule): its box starts at the 16-byte boundary below the block and is 240 bytes wide, and
// the decoder starts at the remainder inside the row.  Rows must be 16-byte multiples (QwArgs::staged says
// whether the host could build the byte map; otherwise the producers read global memory as before).
template <int QT>
struct MmqStage {
  // bytes of 256 values of one row, and bytes fetched per row (16-byte multiples; never a multiple of 128, which
  // would put every row of the box on the same shared-memory banks)
  static constexpr int SB = QT == QT_Q6_K ? 210 : QT == QT_Q8_0 ? 272 : QT == QT_FP8B ? 256 : 144;
  static constexpr int BOX = QT == QT_Q6_K ? 240 : (QT == QT_Q8_0 || QT == QT_FP8B) ? 272 : 144;
  static constexpr int BYTES = GEMM_BM * BOX;
  static constexpr int RING = BOX == 144 ? 6 : BOX == 240 ? 4 : 3;  // boxes per CTA (108 / 120 / 102 KB); see MmqRing
};
// bytes fetched per row for a packed format (host side)
inline int mmq_box_bytes(int qtype) { return qtype == QT_Q6_K ? 240 : (qtype == QT_Q8_0 || qtype == QT_FP8B) ? 272 : 144; }
// boxes per CTA: the 272-byte formats keep two with 128-token tiles, which leaves room for a deeper stage ring
template <int TN, int QT>
struct MmqRing {
  static constexpr int value = (TN >= 128 && MmqStage<QT>::BOX == 272) ? 2 : MmqStage<QT>::RING;
};
template <int TN, int QT>
struct MmqStaged {
  static constexpr bool value = QT != QT_BF16;
};
// Packed weights: the decoded weight tile (the A operand, 128 rows x 64 values per k-block) never touches shared
// memory.  The producer warps write it into tensor memory (tcgen05.st: row = TMEM lane, two bf16 per 32-bit column)
// and the MMA takes A from there; a stage of the ring is then one activation tile in shared memory plus 32 TMEM
// columns.  Shared-memory bandwidth is what bounds this kernel at decode sizes (a 16 KB tile written by the decoders
// and read again by the tensor core, every k-block, next to the packed boxes and the activation tiles), so taking the
// A tile off that path is worth more than any saving in the decode arithmetic.
template <int TN, int QT>
struct GemmStages {
  static constexpr bool A_IN_TMEM = QT != QT_BF16;
  static constexpr int STAGE_BYTES = A_IN_TMEM ? GemmTile<TN>::B_BYTES : GemmTile<TN>::STAGE_BYTES;
  static constexpr int B_OFFSET = A_IN_TMEM ? 0 : GemmTile<TN>::A_BYTES;  // activation tile inside a stage
  static constexpr int TMEM_A_COLS = GEMM_BK / 2;                         // 32-bit columns of one decoded k-block
  // TMEM: accumulator first, then the A ring; the packed-weight kernel takes all 512 columns (it is alone on its SM).
  // Ring depth: bf16 weights use GemmTile's (the weight stream itself fills the ring).  For packed weights no unit of
  // the pipeline is saturated at decode sizes (decoders, TMA and MMA warps each wait a third of the time on the
  // others): what bounds the k-block rate is the number of k-blocks in flight, so the ring is as deep as tensor
  // memory and shared memory allow, up to 12.
  static constexpr int TMEM_COLS = A_IN_TMEM ? 512 : GemmTile<TN>::TMEM_COLS;
  static constexpr int FIT_TMEM = (512 - GemmTile<TN>::ACC_COLS) / TMEM_A_COLS;
  static constexpr int RING_BYTES = QT == QT_BF16 ? 0 : MmqRing<TN, QT>::value * MmqStage<QT>::BYTES;
  static constexpr int FIT_SMEM = (224 * 1024 - 1024 - 512 - 1024 - RING_BYTES) / (STAGE_BYTES > 0 ? STAGE_BYTES : 1);
  static constexpr int FIT = FIT_TMEM < FIT_SMEM ? FIT_TMEM : FIT_SMEM;
  static constexpr int value = QT == QT_BF16 ? GemmTile<TN>::STAGES : (FIT > 12 ? 12 : FIT);
};
template <int TN, int QT>
constexpr int gemm_smem_bytes() {
  return GemmStages<TN, QT>::value * GemmStages<TN, QT>::STAGE_BYTES + 1024 /*align slack*/ + 512 /*barriers*/ + 1024 /*token scales*/ +
         (MmqStaged<TN, QT>::value ? MmqRing<TN, QT>::value * MmqStage<QT>::BYTES : 0);
}

// Epilogue modes
constexpr int EPI_STORE = 0;      // Y = acc (+bias)
constexpr int EPI_ADD_INTO = 1;   // Y += acc (residual accumulate, bf16 read-modify-write)
constexpr int EPI_ROPE = 3;       // fused qkv projection: RoPE on q/k heads, q -> q_out, k/v -> paged KV cache (RopeArgs)
constexpr int EPI_SWIGLU = 2;     // weight rows interleaved per tile (64 gate rows, then their 64 up rows):
                                  // Y[t, n0/2 + c] = silu(acc[c]) * acc[64 + c], Y has N/2 columns
constexpr int EPI_GEGLU = 4;      // the same with the tanh form of GELU on the gate (Gemma)

// RMSNorm folded into the GEMMs around it.  The norm weight is multiplied into the consuming projection's
// columns when the model is loaded; what remains of the norm is one scalar per token, 1/rms(x_t), which
// commutes with the matrix product and is applied to the accumulator in the consumer's epilogue (before
// bias, RoPE or SiLU).  The producer of x (the row-parallel projection whose epilogue writes the new
// residual stream) adds, for every 128-column tile and token, the sum of squares of what it wrote into one
// 64-bit fixed-point accumulator per token (2^-28 units).  Integer addition is associative, so the total does
// not depend on the order in which the tiles arrive: every rank and every replay computes the same scale.
// Two accumulator arrays alternate; the consumer of one clears the other for the producer that follows it.
constexpr float SUMSQ_FIX = 268435456.f;  // 2^28
// Accumulators of neighbouring tokens are 128 bytes apart: every column tile of a token adds into the same word, and
// atomics on one cache line are performed one after the other; with the tokens on separate lines they proceed in parallel.
constexpr int SUMSQ_STRIDE = 16;  // in 64-bit words
struct NormArgs {
  const unsigned long long* sumsq_in;  // consumer: [T * SUMSQ_STRIDE] fixed-point sums of squares of the token rows of X, or null
  float inv_dim, eps;                  // scale_t = rsqrt(sum_t * inv_dim + eps)
  unsigned long long* clear;           // consumer: accumulator array (same layout) to reset for the next producer, or null
  unsigned long long* sumsq_out;       // producer: accumulator array (same layout) that receives the rows written, or null
};

__device__ __forceinline__ void sumsq_add(unsigned long long* dst, float ss) {
  ss = fminf(ss, 3.0e10f);  // 2^63 / 2^28 with headroom for the other tiles of the row
  atomicAdd(dst, (unsigned long long)(ss * SUMSQ_FIX + 0.5f));
}

__device__ __forceinline__ float sumsq_bf16x8(const uint4 v) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(u[j]);
    s += f.x * f.x + f.y * f.y;
  }
  return s;
}
// sum over the 16 lanes that share bit 4 of the lane id (one token row of a 128-column tile)
__device__ __forceinline__ float half_warp_sum(float v) {
  const unsigned mask = (threadIdx.x & 16) ? 0xFFFF0000u : 0x0000FFFFu;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
  return v;
}

// Sum `splits` fp32 partials for tokens [jb, je) of one tile row: JU tokens x SMAX splits of
// independent L2 loads are in flight per thread; the adds run in split order (reproducible).
template <int JU, int SMAX, class Emit>
__device__ __forceinline__ void splitk_reduce(const float* base, int split_stride, int splits, int jb, int je, Emit emit) {
  for (int j0 = jb; j0 < je; j0 += JU) {
    float v[JU][SMAX];
#pragma unroll
    for (int u = 0; u < JU; ++u)
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
        v[u][s] = (j0 + u < je && s < splits) ? __ldcg(base + (size_t)s * split_stride + (j0 + u) * GEMM_BM) : 0.f;
#pragma unroll
    for (int u = 0; u < JU; ++u) {
      float acc = 0.f;
#pragma unroll
      for (int s = 0; s < SMAX; ++s) acc += v[u][s];
      if (j0 + u < je) emit(j0 + u, acc);
    }
  }
}

// Same reduction with the partials in the shared memory of the cluster's CTAs (CTA s holds split s
// at the same shared-memory offset): `local_addr` is this thread's element of token 0 in its own CTA.
template <int JU, int SMAX, class Emit>
__device__ __forceinline__ void splitk_reduce_dsmem(uint32_t local_addr, int splits, int jb, int je, Emit emit) {
  uint32_t peer[SMAX];
#pragma unroll
  for (int s = 0; s < SMAX; ++s) peer[s] = dsmem_map(local_addr, s < splits ? s : 0);
  for (int j0 = jb; j0 < je; j0 += JU) {
    float v[JU][SMAX];
#pragma unroll
    for (int u = 0; u < JU; ++u)
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
        v[u][s] = (j0 + u < je && s < splits) ? dsmem_ld_f32(peer[s] + (uint32_t)(j0 + u) * (GEMM_BM * 4)) : 0.f;
#pragma unroll
    for (int u = 0; u < JU; ++u) {
      float acc = 0.f;
#pragma unroll
      for (int s = 0; s < SMAX; ++s) acc += v[u][s];
      if (j0 + u < je) emit(j0 + u, acc);
    }
  }
}

// bf16 tile [ntok][128 rows] in shared memory -> Y rows with 16-byte stores (128 threads, tid 0..127).
// With ssq_out, the sum of squares of every row written (its 128 columns) is added to ssq_out[t_first + t].
__device__ __forceinline__ void store_tile_rows(const uint8_t* stage, int ntok, int t_first, int n0, int N,
                                                __nv_bfloat16* Y, int ldY, int epi_mode, int tid,
                                                unsigned long long* ssq_out = nullptr) {
  const int chunk = tid & 15, trow = tid >> 4;
  const bool col_ok = n0 + chunk * 8 < N;
  if (!col_ok && ssq_out == nullptr) return;
  const bool add = epi_mode == EPI_ADD_INTO;
  // eight rows per thread and pass: when the tile is added into Y, the eight reads of Y are issued together
  // (one memory latency per pass instead of one per row)
  for (int tb = trow; tb < ntok; tb += 64) {
    uint4 prev[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = tb + 8 * i;
      prev[i] = make_uint4(0, 0, 0, 0);
      if (add && col_ok && t < ntok) prev[i] = *reinterpret_cast<const uint4*>(Y + (size_t)(t_first + t) * ldY + n0 + chunk * 8);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = tb + 8 * i;
      if (t >= ntok) break;  // the 16 lanes of a row share t
      float ss = 0.f;
      if (col_ok) {
        uint4 v = *reinterpret_cast<const uint4*>(stage + t * 256 + chunk * 16);
        if (add) {
          uint32_t a[4] = {v.x, v.y, v.z, v.w};
          const uint32_t c[4] = {prev[i].x, prev[i].y, prev[i].z, prev[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 fa = unpack_bf16x2(a[j]), fc = unpack_bf16x2(c[j]);
            a[j] = pack_bf16x2(fa.x + fc.x, fa.y + fc.y);
          }
          v = make_uint4(a[0], a[1], a[2], a[3]);
        }
        *reinterpret_cast<uint4*>(Y + (size_t)(t_first + t) * ldY + n0 + chunk * 8) = v;
        ss = sumsq_bf16x8(v);
      }
      if (ssq_out != nullptr) {
        ss = half_warp_sum(ss);
        if (chunk == 0) sumsq_add(ssq_out + (size_t)(t_first + t) * SUMSQ_STRIDE, ss);
      }
    }
  }
}

// SwiGLU epilogue: the staged tile holds 64 gate columns followed by the 64 matching up columns of each
// token; writes the 64 activations with 16-byte stores (128 threads: 8 chunks x 16 token rows per pass).
// gelu: act(g) = g * sigmoid(2 sqrt(2/pi) (g + 0.044715 g^3)) (= 0.5 g (1 + tanh(...))) instead of g * sigmoid(g).
__device__ __forceinline__ float glu_gate(float g, bool gelu) {
  const float z = gelu ? 1.5957691216057308f * (g + 0.044715f * g * g * g) : g;
  return g / (1.f + __expf(-z));
}

__device__ __forceinline__ void store_tile_rows_swiglu(const uint8_t* stage, int ntok, int t_first, int n0,
                                                       __nv_bfloat16* Y, int ldY, int tid, bool gelu) {
  const int chunk = tid & 7, trow = tid >> 3;
  for (int t = trow; t < ntok; t += 16) {
    const uint4 g = *reinterpret_cast<const uint4*>(stage + t * 256 + chunk * 16);
    const uint4 u = *reinterpret_cast<const uint4*>(stage + t * 256 + 128 + chunk * 16);
    const uint32_t gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gv[j]), b = unpack_bf16x2(uv[j]);
      o[j] = pack_bf16x2(glu_gate(a.x, gelu) * b.x, glu_gate(a.y, gelu) * b.y);
    }
    *reinterpret_cast<uint4*>(Y + (size_t)(t_first + t) * ldY + (n0 >> 1) + chunk * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// RoPE + KV-write epilogue of the fused qkv projection (EPI_ROPE): a 128-row tile is exactly one head
// (head_dim 128).  Query heads are rotated and written to q_out [T, nq, 128]; key heads are rotated and
// written into the paged cache at the token's slot; value heads are written as they are.  Same
// arithmetic as qk_rope_kvwrite_kernel (table of cos | sin per position, both pairings), bf16 KV only.
struct RopeArgs {
  const int* positions;   // [T]
  const int* slots;       // [T] block * page + offset, < 0 = do not write K/V
  const float* cos_sin;   // [max_pos, rot]: cos for the rot/2 pairs, then sin
  int max_pos, rot, pairing /*0 split-half, 1 adjacent*/;
  int nq, nkv, page, num_blocks;
  __nv_bfloat16* q_out;   // [T, nq, 128]
  __nv_bfloat16* kv_data; // layer base: [blocks, nkv, 2, page, 128]
};

__device__ __forceinline__ void store_tile_rows_rope(const uint8_t* stage, int ntok, int t_first, int n0, const RopeArgs& ro,
                                                     int tid) {
  const int head = n0 >> 7;
  const bool is_q = head < ro.nq, is_k = !is_q && head < ro.nq + ro.nkv;
  const int chunk = tid & 15, trow = tid >> 4;
  const int half = ro.rot >> 1;
  for (int t = trow; t < ntok; t += 8) {
    const int tok = t_first + t;
    const uint4 raw = *reinterpret_cast<const uint4*>(stage + t * 256 + chunk * 16);
    const uint32_t rv[4] = {raw.x, raw.y, raw.z, raw.w};
    float x[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(rv[j]);
      x[2 * j] = f.x;
      x[2 * j + 1] = f.y;
    }
    if (is_q || is_k) {
      int p = ro.positions[tok];
      p = p < 0 ? 0 : (p >= ro.max_pos ? ro.max_pos - 1 : p);
      const float* cs = ro.cos_sin + (size_t)p * ro.rot;
      if (ro.pairing == 0) {
        const uint4 praw = *reinterpret_cast<const uint4*>(stage + t * 256 + (chunk ^ 8) * 16);
        const uint32_t pv[4] = {praw.x, praw.y, praw.z, praw.w};
        const bool first = chunk < 8;
        const int pair0 = (chunk & 7) * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 o = unpack_bf16x2(pv[j]);
          const float c0 = cs[pair0 + 2 * j], s0 = cs[half + pair0 + 2 * j];
          const float c1 = cs[pair0 + 2 * j + 1], s1 = cs[half + pair0 + 2 * j + 1];
          const float v0 = x[2 * j], v1 = x[2 * j + 1];
          x[2 * j] = first ? (v0 * c0 - o.x * s0) : (v0 * c0 + o.x * s0);
          x[2 * j + 1] = first ? (v1 * c1 - o.y * s1) : (v1 * c1 + o.y * s1);
        }
      } else {
        const int pair0 = chunk * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float c = cs[pair0 + j], s = cs[half + pair0 + j];
          const float a = x[2 * j], b = x[2 * j + 1];
          x[2 * j] = a * c - b * s;
          x[2 * j + 1] = b * c + a * s;
        }
      }
    }
    const uint4 o = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
    if (is_q) {
      *reinterpret_cast<uint4*>(ro.q_out + ((size_t)tok * ro.nq + head) * 128 + chunk * 8) = o;
    } else {
      const int slot = ro.slots[tok];
      if (slot >= 0) {
        const int kvh = is_k ? head - ro.nq : head - ro.nq - ro.nkv;
        const int blk = slot / ro.page, off = slot % ro.page;
        if (blk < ro.num_blocks) {
          const size_t row = (((size_t)blk * ro.nkv + kvh) * 2 + (is_k ? 0 : 1)) * ro.page + off;
          *reinterpret_cast<uint4*>(ro.kv_data + row * 128 + chunk * 8) = o;
        } else if (chunk == 0) {
          oxb_report(OXB_BAD_SLOT, slot);  // never write outside the pool
        }
      }
    }
  }
}

// Grouped (per-expert) launches: blockIdx.z selects the group instead of a token tile.  Group z uses
// weight rows [z*w_rows, z*w_rows + N), activation rows [z*x_rows, z*x_rows + T) (x_rows = 0: all
// groups share X), writes Y + z*y_stride, and is skipped entirely when its row of per-token scales
// is all zero (an expert no token was routed to) — so idle experts cost no weight traffic.
struct GroupArgs {
  int enabled;
  int w_rows, x_rows;
  long long y_stride;
  const float* scale;  // [groups, scale_ld] or null (never skip)
  int scale_ld;
  int l2_prefetch_kb;  // weight k-blocks to request into the L2 before the grid dependency (any launch)
  // Token-gathered groups (mixture-of-experts dispatch): group z multiplies activation rows
  // [row_offsets[z], row_offsets[z + 1]) (device array, written by the upstream kernel) and writes the same rows
  // of Y; blockIdx.z = z * t_tiles + token tile, and a CTA whose tile lies past the group's rows leaves at once.
  const int* row_offsets;
  int t_tiles;
};

// 16 accumulator columns of this warp's TMEM lanes
__device__ __forceinline__ void tmem_ld16_now(uint32_t taddr, uint32_t* r) {
  tmem_ld16(taddr, r);
  tmem_ld_wait();
}

#ifdef OXB_MMQ_TRACE
// Phase trace of one CTA of the packed-weight GEMM (cycles spent in each wait, per role), per translation unit
static __device__ long long g_oxb_mmq_trace[32];
#define OXB_TR_DECL long long tr_w0 = 0, tr_w1 = 0, tr_w2 = 0; const long long tr_begin = clock64();
#define OXB_TR_WAIT(acc, expr) [&]() { const long long t_ = clock64(); const bool ok_ = (expr); acc += clock64() - t_; return ok_; }()
#define OXB_TR_STORE(slot) if (MMQ && blockIdx.x == gridDim.x / 2 && blockIdx.y == 0 && blockIdx.z == 0) { \
    g_oxb_mmq_trace[(slot) * 4 + 0] = clock64() - tr_begin; g_oxb_mmq_trace[(slot) * 4 + 1] = tr_w0; \
    g_oxb_mmq_trace[(slot) * 4 + 2] = tr_w1; g_oxb_mmq_trace[(slot) * 4 + 3] = tr_w2; }
#define OXB_TR_BEGIN const long long tr_t_ = clock64();
#define OXB_TR_END(acc) acc += clock64() - tr_t_;
#else
#define OXB_TR_DECL
#define OXB_TR_WAIT(acc, expr) (expr)
#define OXB_TR_STORE(slot)
#define OXB_TR_BEGIN
#define OXB_TR_END(acc)
#endif

// QT == QT_BF16: both operands arrive by TMA.  Any other QT: the weight tile is decoded by the producer warps from
// packed blocks into tensor memory (see mmq_producer.cuh) and only the activations (and the packed boxes) use TMA.
template <int TN, int QT>
__global__ void __launch_bounds__(QT == QT_BF16 ? GEMM_THREADS : GEMM_THREADS_MMQ, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 __nv_bfloat16* __restrict__ Y, const float* __restrict__ bias, int N, int T, int K, int ldY,
                 int splits, float* __restrict__ ws, int* __restrict__ counters, int epi_mode, const ArArgs ar,
                 const QwArgs qw, const GroupArgs gr, const RopeArgs ro, const NormArgs nm) {
  constexpr bool MMQ = QT != QT_BF16;
  const bool gathered = gr.enabled && gr.row_offsets != nullptr;
  const int zg = gr.enabled ? (gathered ? (int)blockIdx.z / gr.t_tiles : (int)blockIdx.z) : 0;
  int g_row0 = 0;  // first activation / output row of this group (gathered groups)
  if (gathered) {
    pdl_wait();  // the row lists come from the upstream kernel
    g_row0 = gr.row_offsets[zg];
    T = gr.row_offsets[zg + 1] - g_row0;  // this group's own row count
    if (((int)blockIdx.z % gr.t_tiles) * TN >= T) {
      pdl_launch_dependents();
      return;
    }
  }
  if (gr.enabled && !gathered && gr.scale != nullptr) {
    // the routing weights come from the upstream kernel
    pdl_wait();
    int any = 0;
    for (int t = threadIdx.x; t < T; t += blockDim.x) any |= gr.scale[(size_t)zg * gr.scale_ld + t] != 0.f;
    if (!__syncthreads_or(any)) {
      pdl_launch_dependents();
      return;
    }
  }
  Y += gathered ? (size_t)g_row0 * ldY : (size_t)zg * gr.y_stride;
  using Cfg = GemmTile<TN>;
  constexpr int STAGES = GemmStages<TN, QT>::value;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using St = GemmStages<TN, QT>;
  constexpr int STAGE_BYTES = St::STAGE_BYTES;
  constexpr bool STAGED = MmqStaged<TN, QT>::value;
  constexpr int PRING = STAGED ? MmqRing<TN, QT>::value : 0;
  // layout: stage ring | ring of packed boxes | barriers (512 B) | token scales.  The epilogue stages its tiles from
  // the start of the buffer and may run over both rings, which are idle by then.
  uint8_t* packed_buf = smem + STAGES * STAGE_BYTES;                                             // [PRING][128][BOX]
  uint8_t* bars = packed_buf + PRING * MmqStage<QT>::BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(bars);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* ticket = const_cast<int*>(abort_flag) + 1;
  // a producer group may run at most STAGES k-blocks ahead of the slowest one; with more groups than stages it could
  // be two uses of a stage ahead, which the one-bit phase of the stage's barrier cannot tell apart
  static_assert(!MMQ || STAGES >= MMQ_GROUPS, "the stage ring must be at least as deep as the number of producer groups");
  static_assert(STAGES * STAGE_BYTES + PRING * MmqStage<QT>::BYTES >= TN * GEMM_BM * 6,
                "the epilogue stages fp32 partials and a bf16 tile in the ring memory");
  static_assert(STAGES <= 12 && PRING <= 8, "barrier block layout");
  uint64_t* packed_full = reinterpret_cast<uint64_t*>(bars + 256);  // [PRING <= 8] (STAGED only)
  uint64_t* packed_empty = packed_full + 8;                        // [PRING <= 8]
  float* tok_scale = reinterpret_cast<float*>(bars + 512);         // [TN]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Plain launches with several token tiles walk the tile grid token-major: consecutive CTAs (one wave holds 148 of
  // them) share a weight tile and differ in the token tile, so a wave touches few weight tiles and all activation
  // tiles, both of which then stay in the L2, instead of every weight tile of the matrix in every wave.
  int tile_n = blockIdx.x, tile_t = blockIdx.z;
  if (!gr.enabled && gridDim.z > 1 && gridDim.y == 1) {
    const int lin = blockIdx.z * gridDim.x + blockIdx.x;
    tile_n = lin / (int)gridDim.z;
    tile_t = lin % (int)gridDim.z;
  }
  const int n0 = tile_n * GEMM_BM;
  const int split = blockIdx.y;
  const int t0 = gathered ? ((int)blockIdx.z % gr.t_tiles) * TN : (gr.enabled ? 0 : tile_t * TN);
  const int w_row0 = n0 + zg * gr.w_rows;  // first weight row of this tile in the (stacked) matrix
  const int x_row0 = gathered ? g_row0 + t0 : t0 + zg * gr.x_rows;
  const int kb_total = (K + GEMM_BK - 1) / GEMM_BK;
  const int kb_begin = (int)((long long)split * kb_total / splits);
  const int kb_end = (int)((long long)(split + 1) * kb_total / splits);
  const int nkb = kb_end - kb_begin;
  // launched as clusters of `splits` CTAs along y: split-K reduces through distributed shared memory
  const bool csplit = splits > 1 && cluster_nctarank() == (uint32_t)splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], MMQ ? 1 + 4 : 1);  // TMA expect_tx arrival (+ one per producer warp of a group)
      mbar_init(&empty[i], 1);
    }
    mbar_init(accum, 1);
    if constexpr (STAGED) {
      for (int i = 0; i < PRING; ++i) {
        mbar_init(&packed_full[i], 1);
        mbar_init(&packed_empty[i], 4 * MMQ_GROUPS);  // one arrival per producer warp
      }
    }
    *abort_flag = 0;
    ticket[0] = 0;
    mbar_fence_init();
  }
  if (warp == GEMM_WARP_MMA) {
    tmem_alloc(tmem_slot, St::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The next kernel may start its own set-up now.  (Packed weights: only after this CTA's registers have been
  // moved between its warpgroups, see below, so that no CTA of the next kernel can take what a warpgroup released.)
  if constexpr (!MMQ) pdl_launch_dependents();

  // Packed weights: 768 threads leave 80 registers each.  The decoders need few, the epilogue many: the second
  // warpgroup (TMA, MMA, idle) and the producers hand registers back, the epilogue warpgroup takes exactly what they
  // released (a CTA can only redistribute its own launch allocation; the request waits for the other warpgroups'
  // releases, which are the first instruction of their branches).  Each budget is set at the top of its branch.
  if (warp >= 4 && warp < GEMM_WARP_PRODUCER0) {
    if constexpr (MMQ) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(MMQ_REGS_CONTROL));
  // The two control warps run their loops with all 32 lanes (waits, counters and addresses are then warp-uniform and
  // can live in the uniform datapath, which is where TMA and MMA instructions take their operands from); one elected
  // lane issues.  With a single thread running the whole loop every operand had to be moved over per instruction, and
  // the serial latency of that thread's instruction stream, several hundred cycles per k-block, bounded the
  // packed-weight kernel whatever the decoders did.
  if (warp == GEMM_WARP_TMA) {
    // ---------------- TMA producer
    OXB_TR_DECL
    const bool leader = elect_one();
    const uint64_t pol_w = l2_policy_evict_first();  // weights are read once per step
    const uint64_t pol_x = l2_policy_evict_last();   // activations are re-read by every CTA
    const int npre = nkb < STAGES ? nkb : STAGES;
    if (leader) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      // Weights are static: the first ring's worth of weight tiles is requested before waiting for
      // the upstream kernel, so the weight stream overlaps the previous kernel's tail.
      for (int i = 0; i < npre; ++i) {
        uint8_t* sA = smem + i * STAGE_BYTES;
        if constexpr (MMQ) {
          mbar_expect_tx(&full[i], Cfg::B_BYTES);
        } else {
          mbar_expect_tx(&full[i], Cfg::STAGE_BYTES);
          tma_load_2d_hint(sA, &tmW, &full[i], (kb_begin + i) * GEMM_BK, w_row0, pol_w);
        }
      }
      if constexpr (!MMQ) {
        // ... and the rest of this CTA's weight slice is requested into the L2, where the main loop
        // will find it once the activations are there.
        const int npf = nkb < gr.l2_prefetch_kb ? nkb : gr.l2_prefetch_kb;
        for (int i = npre; i < npf; ++i) tma_prefetch_l2_2d(&tmW, (kb_begin + i) * GEMM_BK, w_row0);
      }
    }
    pdl_wait();  // activations come from the upstream kernel
    if (leader) {
      for (int i = 0; i < npre; ++i) {
        uint8_t* sB = smem + i * STAGE_BYTES + St::B_OFFSET;
        tma_load_2d_hint(sB, &tmX, &full[i], (kb_begin + i) * GEMM_BK, x_row0, pol_x);
      }
    }
    int st = npre == STAGES ? 0 : npre;  // stage of k-block npre
    uint32_t ph = 0;                     // parity of the completion of empty[st] that frees it for its next use
    for (int i = npre; i < nkb; ++i) {
      const bool ok = OXB_TR_WAIT(tr_w0, mbar_wait_bounded(&empty[st], ph, abort_flag, OXB_TIMEOUT_TMA_EMPTY, blockIdx.x));
      if (!__all_sync(0xffffffffu, ok)) break;
      if (leader) {
        uint8_t* sA = smem + st * STAGE_BYTES;
        uint8_t* sB = sA + St::B_OFFSET;
        if constexpr (MMQ) {
          mbar_expect_tx(&full[st], Cfg::B_BYTES);
        } else {
          mbar_expect_tx(&full[st], Cfg::STAGE_BYTES);
          tma_load_2d_hint(sA, &tmW, &full[st], (kb_begin + i) * GEMM_BK, w_row0, pol_w);
        }
        tma_load_2d_hint(sB, &tmX, &full[st], (kb_begin + i) * GEMM_BK, x_row0, pol_x);
      }
      if (++st == STAGES) {
        st = 0;
        ph ^= 1;
      }
    }
    if (leader) { OXB_TR_STORE(0) }
  } else if (warp == GEMM_WARP_MMA) {
    // ---------------- MMA issuer
    OXB_TR_DECL
    const bool leader = elect_one();
    constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, TN);
    const uint32_t smem_base = smem_u32(smem);
    int st = 0;
    uint32_t ph = 0;
    for (int i = 0; i < nkb; ++i) {
      const bool ok = OXB_TR_WAIT(tr_w0, mbar_wait_bounded(&full[st], ph, abort_flag, OXB_TIMEOUT_TMA_FULL, blockIdx.x));
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      if (leader) {
        const uint32_t a_addr = smem_base + st * STAGE_BYTES;
        const uint64_t adesc = umma_desc_k_sw128(a_addr);
        const uint64_t bdesc = umma_desc_k_sw128(a_addr + St::B_OFFSET);
        {
          OXB_TR_BEGIN
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // advance 16 bf16 = 32 bytes inside the swizzle row: +2 in the (addr >> 4) field; in TMEM 16 bf16 = 8 columns
            if constexpr (MMQ)
              umma_bf16_ts(tmem_base, tmem_base + Cfg::ACC_COLS + st * St::TMEM_A_COLS + 8 * k, bdesc + 2 * k, idesc,
                           (i > 0 || k > 0) ? 1u : 0u);
            else
              umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          OXB_TR_END(tr_w1)
        }
        {
          OXB_TR_BEGIN
          umma_commit(&empty[st]);  // frees the stage when these MMAs have read it
          OXB_TR_END(tr_w2)
        }
      }
      if (++st == STAGES) {
        st = 0;
        ph ^= 1;
      }
    }
    if (leader) {
      umma_commit(accum);
      // The issuing lane alone polls for the end of the MMAs, then the warp releases the four epilogue warps from a
      // named barrier: 128 threads spinning on a shared-memory barrier for the whole main loop take issue slots and
      // shared-memory cycles from the warps that feed the tensor core.  (The wait is bounded; on a timeout the abort
      // flag is set and the barrier is released all the same.)
      mbar_wait_bounded(accum, 0, abort_flag, OXB_TIMEOUT_ACCUM, blockIdx.x);
      OXB_TR_STORE(1)
    }
    __syncwarp();
    asm volatile("bar.arrive 3, 160;" ::: "memory");
  }
    __syncwarp();
    if (csplit) {
      cluster_sync_all();
      cluster_sync_all();
    }
  } else if (warp >= GEMM_WARP_PRODUCER0) {
    if constexpr (MMQ) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(MMQ_REGS_PRODUCER));
    // ---------------- dequant producers (MMQ only): MMQ_GROUPS groups of 128 threads; in each, thread r decodes weight row
    // n0 + r.  Group g takes k-blocks g, g + MMQ_GROUPS, ... (each stage's barrier expects the four warps of ONE
    // group), so MMQ_GROUPS k-blocks are being decoded at any time.
    if constexpr (MMQ) {
      OXB_TR_DECL
      const int grp = (threadIdx.x - 32 * GEMM_WARP_PRODUCER0) >> 7;
      const int r = (threadIdx.x - 32 * GEMM_WARP_PRODUCER0) & 127;
      const int n = n0 + r;
      const uint8_t* rowp = qw.w + ((size_t)zg * gr.w_rows + (size_t)(n < N ? n : 0)) * qw.row_bytes;
      // Fallback when the packed rows cannot be mapped for TMA (rows or base not 16-byte multiples, K not a multiple
      // of 256): each thread walks its own packed row in global memory.  Addresses are clamped to valid blocks;
      // out-of-range results are zeroed afterwards.
      const int kb_last = (K / GEMM_BK) - 1;
      auto decode = [&](int kb, uint32_t* v) {
        const int kbc = kb < kb_last ? kb : kb_last;
        dequant64<QT>(rowp, kbc * GEMM_BK, qw, n < N ? n : 0, v);
      };
      auto mask = [&](int kb, uint32_t* v) {
        if (!(n < N && kb <= kb_last)) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
      };
      // this thread's row of stage st in TMEM: lane = row (the warp's lane quarter is warp % 4), 32 columns per stage
      const uint32_t a_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + Cfg::ACC_COLS;
      auto wait_slot = [&](int i) -> bool {
        const int st = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        // warp-uniform verdict: the warp-level synchronisation below must be reached by all 32 lanes or none
        const bool ok = OXB_TR_WAIT(tr_w0, __all_sync(0xffffffffu, mbar_wait_bounded(&empty[st], ph ^ 1, abort_flag,
                                                                                    OXB_TIMEOUT_TMA_EMPTY, blockIdx.x)));
        if (ok) tc_fence_after();  // the MMAs that read this slot are done: order this thread's TMEM stores after them
        return ok;
      };
      auto signal_slot = [&](int i) {
        tmem_st_wait();     // this thread's stores have landed in TMEM
        tc_fence_before();  // ... and are ordered before the MMA thread's reads through the barrier
        __syncwarp();       // the warp's 32 rows are written: one arrival per warp instead of 32
        if (lane == 0) mbar_arrive(&full[i % STAGES]);
      };
      auto publish = [&](int i, const uint32_t* v) -> bool {  // a k-block decoded into registers beforehand
        if (!wait_slot(i)) return false;
        const uint32_t dst = a_lane + (i % STAGES) * St::TMEM_A_COLS;
#pragma unroll
        for (int c = 0; c < 8; ++c) tmem_st4(dst + 4 * c, v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        signal_slot(i);
        return true;
      };
      // staged form: wait for the ring slot first, then decode the row out of shared memory straight into it
      auto publish_from = [&](int i, const uint8_t* srow, int kb) -> bool {
        if (!wait_slot(i)) return false;
        const uint32_t dst = a_lane + (i % STAGES) * St::TMEM_A_COLS;
        auto put = [&](int c, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) { tmem_st4(dst + 4 * c, w0, w1, w2, w3); };
        {
          OXB_TR_BEGIN
          // No branch on the row index here: tcgen05.st is a warp-wide instruction (all 32 lanes must execute the same
          // one), and a tile whose last rows lie past N has warps with both kinds of lanes.  Rows past N decode whatever
          // the box holds there (zeros past the end of the matrix, the next expert's rows in a stacked one); the
          // epilogue never stores them.
          if constexpr (QT == QT_FP8B)  // scales are indexed by the absolute row and channel
            dequant64_chunks<QT>(srow - (size_t)(kb & ~3) * GEMM_BK, kb * GEMM_BK, qw, n < N ? n : 0, put);
          else
            dequant64_chunks<QT>(srow, (kb & 3) * GEMM_BK, qw, 0, put);
          OXB_TR_END(tr_w2)
        }
        signal_slot(i);
        return true;
      };
      bool staged_done = false;
      if constexpr (STAGED) if (qw.staged) {
        staged_done = true;
        constexpr int SB = MmqStage<QT>::SB, BOX = MmqStage<QT>::BOX, PBYTES = MmqStage<QT>::BYTES;
        // Packed super-blocks arrive by TMA (tmW maps the packed rows as bytes): thread 192 keeps PRING - 1
        // boxes in flight while one is decoded; all producers decode their own row out of shared memory and
        // every warp releases a box when it is done with it.  Weights are static, so none of this waits for
        // the upstream kernel.
        const int sb_begin = kb_begin >> 2, sb_end = (kb_end + 3) >> 2;  // super-blocks touched by [kb_begin, kb_end)
        const int nsb = sb_end - sb_begin;
        auto sb_at = [&](int j) { return sb_begin + j; };  // j-th super-block of this CTA
        auto issue = [&](int j) {  // j-th super-block in processing order -> box j % PRING
          const int b = j % PRING;
          mbar_expect_tx(&packed_full[b], PBYTES);
          tma_load_2d(packed_buf + b * PBYTES, &tmW, &packed_full[b], ((sb_at(j) * SB) & ~15) >> 2, w_row0);
        };
        const bool issuer = r == 0 && grp == 0;
        if (issuer) {
          tma_prefetch_desc(&tmW);
          for (int j = 0; j < PRING && j < nsb; ++j) issue(j);
        }
        bool alive = true;
        for (int j = 0; j < nsb; ++j) {
          const int b = j % PRING;
          // the box of super-block j - 1 is refilled as soon as every warp has let go of it
          if (issuer && alive && j >= 1 && j - 1 + PRING < nsb) {
            if (OXB_TR_WAIT(tr_w1, mbar_wait_bounded(&packed_empty[(j - 1) % PRING], ((j - 1) / PRING) & 1, abort_flag,
                                                     OXB_TIMEOUT_TMA_EMPTY, blockIdx.x)))
              issue(j - 1 + PRING);
          }
          if (alive)
            alive = OXB_TR_WAIT(tr_w1, __all_sync(0xffffffffu, mbar_wait_bounded(&packed_full[b], (j / PRING) & 1, abort_flag,
                                                                                 OXB_TIMEOUT_TMA_FULL, blockIdx.x)));
          if (alive) {
            const int sb = sb_at(j);
            const uint8_t* srow = packed_buf + b * PBYTES + r * BOX + ((sb * SB) & 15);
            const int kb0 = max(kb_begin, sb * 4), kb1 = min(kb_end, sb * 4 + 4);
            for (int kb = kb0; kb < kb1 && alive; ++kb) {
              const int seq = kb - kb_begin;  // the ring's sequence number
              if (seq % MMQ_GROUPS != grp) continue;  // another group's k-block
              alive = publish_from(seq, srow, kb);
            }
          }
          __syncwarp();  // the warp's reads of the box are done (alive or not, so that the issuer never waits in vain)
          if (lane == 0) mbar_arrive(&packed_empty[b]);
        }
      }
      if (!staged_done) {
        // group g takes k-blocks g, g + MMQ_GROUPS, ...; a block is decoded into registers BEFORE the thread waits for
        // its ring slot, so that the global loads overlap the tensor core's work on the slots still in use
        for (int i = grp; i < nkb; i += MMQ_GROUPS) {
          uint32_t v0[32];
          decode(kb_begin + i, v0);
          mask(kb_begin + i, v0);
          if (!publish(i, v0)) break;
        }
      }
      if (r == 0) { OXB_TR_STORE(2 + grp) }
    }
    __syncwarp();
    if (csplit) {
      cluster_sync_all();
      cluster_sync_all();
    }
  } else {
    if constexpr (MMQ) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(MMQ_REGS_EPILOGUE));
      pdl_launch_dependents();
    }
    // ---------------- epilogue: warps 0..3 own TMEM lane quarters (warp % 4)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // row inside the 128-row tile
    const int n = n0 + row;
    const int etid = threadIdx.x;
    pdl_wait();  // everything below reads or writes global memory shared with the upstream kernel
    const bool use_nm = nm.sumsq_in != nullptr;
    if (use_nm) {
      // 1/rms of every token of this tile; computed while the MMAs run, published by the barrier below
      for (int j = etid; j < TN; j += 128) {
        const float s = t0 + j < T ? (float)__ldcg(nm.sumsq_in + (size_t)(t0 + j) * SUMSQ_STRIDE) * (1.f / SUMSQ_FIX) : 0.f;
        tok_scale[j] = rsqrtf(s * nm.inv_dim + nm.eps);
      }
    }
    if (nm.clear != nullptr && tile_n == 0 && blockIdx.y == 0) {
      // the accumulator that the next producer adds into: its last reader finished before this grid's dependency
      const int tt = gr.enabled ? T : min(TN, T - t0);
      for (int j = etid; j < tt; j += 128) nm.clear[(size_t)(t0 + j) * SUMSQ_STRIDE] = 0ull;
    }
    unsigned long long* const ssq_dst = nm.sumsq_out;
    asm volatile("bar.sync 3, 160;" ::: "memory");  // released by the MMA warp once the accumulator is complete
    // agree on one verdict for all 128 epilogue threads before any further named barrier
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 0) {
      ticket[1] = (*abort_flag == 0);
      ticket[2] = ar.world > 0 ? ar.ctrl[0] : 0;  // call counter of this collective (buffer parity, epoch)
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = ticket[1] != 0;
    tc_fence_after();
    const float b = (bias != nullptr && n < N) ? bias[n] : 0.f;
    const int tile_id = blockIdx.z * gridDim.x + blockIdx.x;  // (unique per CTA of a split group in every launch mode)
    const bool use_ar = ar.world > 0;
    const int tvalid = min(TN, T - t0);
    // 16-byte output rows: the tile goes through shared memory as bf16 [token][128 rows] and leaves
    // with coalesced vector stores (a TMEM lane holds ONE output column, so direct stores would be
    // 2-byte writes strided by ldY).
    const bool vec_ok = (N % 8 == 0) && (ldY % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    if (splits == 1) {
      if (ok && (use_ar || vec_ok)) {
        __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem);  // the pipeline memory is idle now
        const float badd = use_ar ? 0.f : b;
#pragma unroll 1
        for (int c = 0; c < TN / 16; ++c) {
          uint32_t r[16];
          tmem_ld16_now(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16, r);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float sc = use_nm ? tok_scale[c * 16 + j] : 1.f;
            stage[(c * 16 + j) * GEMM_BM + row] = __float2bfloat16(__uint_as_float(r[j]) * sc + badd);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (use_ar) {
          ar_exchange(ar, smem, ticket[2], tile_id, n0, t0, tvalid, N, Y, ldY, abort_flag, etid, ssq_dst);
        } else if (epi_mode == EPI_SWIGLU || epi_mode == EPI_GEGLU) {
          store_tile_rows_swiglu(smem, tvalid, t0, n0, Y, ldY, etid, epi_mode == EPI_GEGLU);
        } else if (epi_mode == EPI_ROPE) {
          store_tile_rows_rope(smem, tvalid, t0, n0, ro, etid);
        } else {
          store_tile_rows(smem, tvalid, t0, n0, N, Y, ldY, epi_mode, etid, ssq_dst);
        }
      } else if (ok) {
#pragma unroll 1
        for (int c = 0; c < TN / 16; ++c) {
          uint32_t r[16];
          tmem_ld16_now(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16, r);
          if (n < N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c * 16 + j;
              if (t < T) {
                float v = __uint_as_float(r[j]) * (use_nm ? tok_scale[c * 16 + j] : 1.f) + b;
                __nv_bfloat16* dst = Y + (size_t)t * ldY + n;
                if (epi_mode == EPI_ADD_INTO) v += __bfloat162float(*dst);
                *dst = __float2bfloat16(v);
              }
            }
          }
        }
      }
    } else if (csplit) {
      // Split-K inside a thread-block cluster: the `splits` CTAs of a tile are one cluster.  Each
      // writes its fp32 partial [token][128 rows] into its OWN shared memory, the cluster meets at a
      // hardware barrier, and CTA r sums token slice r straight out of its peers' shared memory
      // (distributed shared memory loads, fixed split order).  No global scratch, atomics or polling.
      float* part = reinterpret_cast<float*>(smem);
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < TN / 16; ++c) {
          uint32_t r[16];
          tmem_ld16_now(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16, r);
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c * 16 + j) * GEMM_BM + row] = __uint_as_float(r[j]);
        }
      }
      cluster_sync_all();
      const int chunk = (tvalid + splits - 1) / splits;
      const int jb = min(tvalid, split * chunk), je = min(tvalid, jb + chunk);
      uint8_t* stage_b = smem + TN * GEMM_BM * 4;
      if (ok) {
        __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(stage_b);
        const float badd = use_ar ? 0.f : b;
        const uint32_t a0 = smem_u32(part + row);
        auto emit = [&](int j, float acc) {
          stage[(j - jb) * GEMM_BM + row] = __float2bfloat16(acc * (use_nm ? tok_scale[j] : 1.f) + badd);
        };
        if (splits <= 2) {
          splitk_reduce_dsmem<8, 2>(a0, splits, jb, je, emit);
        } else if (splits <= 4) {
          splitk_reduce_dsmem<8, 4>(a0, splits, jb, je, emit);
        } else if (splits <= 8) {
          splitk_reduce_dsmem<4, 8>(a0, splits, jb, je, emit);
        } else {
          splitk_reduce_dsmem<2, 16>(a0, splits, jb, je, emit);
        }
      }
      cluster_sync_all();  // every peer has finished reading this CTA's partial
      if (ok && je > jb) {
        if (use_ar) {
          ar_exchange(ar, stage_b, ticket[2], tile_id * splits + split, n0, t0 + jb, je - jb, N, Y, ldY, abort_flag, etid, ssq_dst);
        } else if (epi_mode == EPI_SWIGLU || epi_mode == EPI_GEGLU) {
          store_tile_rows_swiglu(stage_b, je - jb, t0 + jb, n0, Y, ldY, etid, epi_mode == EPI_GEGLU);
        } else if (epi_mode == EPI_ROPE) {
          store_tile_rows_rope(stage_b, je - jb, t0 + jb, n0, ro, etid);
        } else if (vec_ok) {
          store_tile_rows(stage_b, je - jb, t0 + jb, n0, N, Y, ldY, epi_mode, etid, ssq_dst);
        } else if (n < N) {
          const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(stage_b);
          for (int j = jb; j < je; ++j) {
            float v = __bfloat162float(stage[(j - jb) * GEMM_BM + row]);
            __nv_bfloat16* dst = Y + (size_t)(t0 + j) * ldY + n;
            if (epi_mode == EPI_ADD_INTO) v += __bfloat162float(*dst);
            *dst = __float2bfloat16(v);
          }
        }
      }
    } else if (ok) {
      // Split-K through global scratch (launches without a cluster): fp32 partial -> workspace
      // [tile][split][token][row]
      float* my = ws + ((size_t)tile_id * splits + split) * (size_t)(TN * GEMM_BM);
#pragma unroll 1
      for (int c = 0; c < TN / 16; ++c) {
        uint32_t r[16];
        tmem_ld16_now(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16, r);
#pragma unroll
        for (int j = 0; j < 16; ++j) my[(c * 16 + j) * GEMM_BM + row] = __uint_as_float(r[j]);
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // All `splits` CTAs of a tile are co-resident (the host keeps the grid within one wave), so
      // they meet at an arrive counter and then each reduces its own slice of the tile's tokens:
      // the reduction is spread over the CTAs instead of serialised in the last one to arrive.
      int* cnt = counters + 2 * tile_id;  // [arrive, depart]
      if (threadIdx.x == 0) {
        atomicAdd(&cnt[0], 1);
        bool met = false;
        for (unsigned it = 0; it < 20000000u; ++it) {
          if (*reinterpret_cast<volatile int*>(&cnt[0]) >= splits) {
            met = true;
            break;
          }
          if (*abort_flag) break;
          if (it > 64) __nanosleep(32);
        }
        if (!met && !*abort_flag) {
          *abort_flag = 1;
          oxb_report(OXB_TIMEOUT_SPLITK, tile_id);
        }
        ticket[1] = met ? 1 : 0;
        __threadfence();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ticket[1] != 0) {
        const float* base = ws + (size_t)tile_id * splits * (size_t)(TN * GEMM_BM) + row;
        const int chunk = (tvalid + splits - 1) / splits;
        const int jb = min(tvalid, split * chunk), je = min(tvalid, jb + chunk);
        __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem);
        auto emit = [&](int j, float acc) {
          if (use_nm) acc *= tok_scale[j];
          if (use_ar) {
            stage[(j - jb) * GEMM_BM + row] = __float2bfloat16(acc);
          } else if (n < N) {
            acc += b;
            __nv_bfloat16* dst = Y + (size_t)(t0 + j) * ldY + n;
            if (epi_mode == EPI_ADD_INTO) acc += __bfloat162float(*dst);
            *dst = __float2bfloat16(acc);
          }
        };
        if (splits <= 4) {
          splitk_reduce<8, 4>(base, TN * GEMM_BM, splits, jb, je, emit);
        } else if (splits <= 8) {
          splitk_reduce<4, 8>(base, TN * GEMM_BM, splits, jb, je, emit);
        } else {
          splitk_reduce<2, 16>(base, TN * GEMM_BM, splits, jb, je, emit);
        }
        if (use_ar) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (je > jb)
            ar_exchange(ar, smem, ticket[2], tile_id * splits + split, n0, t0 + jb, je - jb, N, Y, ldY, abort_flag, etid, ssq_dst);
        }
        // the last CTA to leave re-arms the counters for the next launch / graph replay
        if (threadIdx.x == 0) {
          if (atomicAdd(&cnt[1], 1) == splits - 1) {
            cnt[1] = 0;
            cnt[0] = 0;
          }
        }
      }
    }
    if (use_ar && threadIdx.x == 0) {
      // the last CTA of the grid advances the call counter (flips the buffer parity)
      __threadfence();
      const int done = atomicAdd(&ar.ctrl[1], 1);
      if (done == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) {
        ar.ctrl[1] = 0;
        __threadfence();
        ar.ctrl[0] = ar.ctrl[0] + 1;
      }
    }
  }

  if (*abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before the CTA exits
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == GEMM_WARP_MMA) tmem_dealloc(tmem_base, St::TMEM_COLS);
}

struct GemmPlan {
  int tn, n_tiles, t_tiles, splits;
  int cluster;  // 1: the splits of a tile form a thread-block cluster (no global scratch needed)
  size_t ws_bytes;
  int n_counters;
};

extern int g_oxb_cluster_splitk;  // 1 = split-K through clusters / distributed shared memory (default)
extern int g_oxb_gemm_prefill_tn;  // 0 = pick the token tile of prefill-sized calls by wave count, 128 / 256 = force

// packed: the packed-weight kernel (one CTA per SM, 128-token tiles at most).  cluster_ok < 0: follow g_oxb_cluster_splitk.  max_ctas > 0 bounds tiles*splits (kernels whose CTAs wait
// for CTAs of other GPUs must be resident all at once).
inline GemmPlan gemm_plan(int T, int N, int K, int splits_hint, int sm_count, int cluster_ok = -1, int max_ctas = 0,
                          bool packed = false, int groups = 1) {
  GemmPlan p;
  if (cluster_ok < 0) cluster_ok = g_oxb_cluster_splitk;
  p.tn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  if (packed && p.tn > 128) p.tn = 128;  // packed weights: 128-token tiles at most (TMEM holds the accumulator and the A ring)
  p.n_tiles = (N + GEMM_BM - 1) / GEMM_BM;
  if (T > 256 && sm_count > 0) {
    // Prefill-sized calls run one CTA per SM in waves; a nearly empty last wave costs a whole tile time.
    // 128-token tiles take half as long as 256-token ones, so compare the wave counts in half-tile units.
    const long long w256 = ((long long)p.n_tiles * ((T + 255) / 256) + sm_count - 1) / sm_count * 2;
    const long long w128 = ((long long)p.n_tiles * ((T + 127) / 128) + sm_count - 1) / sm_count;
    if (g_oxb_gemm_prefill_tn == 128 || (g_oxb_gemm_prefill_tn == 0 && w128 < w256)) p.tn = 128;
  }
  p.t_tiles = (T + p.tn - 1) / p.tn;
  const int kb_total = (K + GEMM_BK - 1) / GEMM_BK;
  int splits = splits_hint;
  if (splits <= 0) {
    // Among the admissible split counts pick the one with the smallest critical path: k-blocks
    // streamed by the busiest SM plus a fixed cost per split for the reduction.  Without clusters
    // the CTAs of a split tile meet at a global counter and must all be resident, which bounds
    // tiles*splits by the SMs' capacity; clusters are co-scheduled by the hardware.
    const int tiles = p.n_tiles * p.t_tiles;
    const int resident = sm_count * (p.tn <= 64 ? 2 : 1);
    // Tiles wider than 64 tokens hold one CTA per SM, and their partials are large: split only
    // within one wave.  Nothing is split once the tiles alone fill the SMs.
    const int wave_cap = p.tn <= 64 ? (1 << 30) : sm_count;
    int capacity = max_ctas > 0 ? max_ctas : (cluster_ok ? wave_cap : resident);
    if (capacity > wave_cap) capacity = wave_cap;
    const int max_by_k = kb_total / 4 > 0 ? kb_total / 4 : 1;  // at least 4 k-blocks (256 columns) per split
    const int epi = p.tn / 32;                                 // k-block equivalents of writing and reducing a partial
    long long best_cost = -1;
    splits = 1;
    const int s_max = p.tn <= 64 ? 16 : 4;  // wide tiles have large partials: a deep split costs more than it streams
    for (int s = 1; s <= s_max && s <= max_by_k && (long long)tiles * s <= capacity && (s == 1 || tiles < sm_count); ++s) {
      const int per_cta = (kb_total + s - 1) / s;
      long long cost;
      if (packed) {
        // One CTA per SM, so the grid runs in waves, and every wave pays the CTA's set-up and epilogue (about a dozen
        // k-block times).  A cluster must fit inside one GPC (18-19 SMs here): s CTAs at a time, the remainder idles.
        const int per_gpc = (sm_count / 8) / s;
        const int slots = per_gpc > 0 ? 8 * per_gpc * s : s;
        const long long ctas = (long long)tiles * groups * s;  // grouped launches: every group has its own tiles
        const int waves = (int)((ctas + (s > 1 ? slots : sm_count) - 1) / (s > 1 ? slots : sm_count));
        cost = (long long)waves * (per_cta + 12) + (s > 1 ? 2 + s / 4 + epi : 0);
      } else {
        const int ctas_on_busiest = (tiles * s + sm_count - 1) / sm_count;
        cost = (long long)ctas_on_busiest * (per_cta + 3) + (s > 1 ? 2 + s / 4 + epi : 0);
      }
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        splits = s;
      }
    }
  }
  if (splits > kb_total) splits = kb_total;
  p.splits = splits;
  p.cluster = (cluster_ok && splits > 1 && splits <= 16) ? 1 : 0;
  const bool scratch = splits > 1 && !p.cluster;
  p.ws_bytes = scratch ? (size_t)p.n_tiles * p.t_tiles * splits * p.tn * GEMM_BM * sizeof(float) : 0;
  p.n_counters = scratch ? 2 * p.n_tiles * p.t_tiles : 0;
  return p;
}

// Largest cluster the kernel instance can be launched with: 16 where the device accepts the
// non-portable size for this footprint, else the portable 8.
template <int TN, int QT>
int gemm_max_cluster() {
  static int cached_dev[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int& cached = cached_dev[dev];
  if (cached) return cached;
  cached = 8;
  auto kfn = gemm_bf16_kernel<TN, QT>;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 16, 1);
    cfg.blockDim = dim3(QT == QT_BF16 ? GEMM_THREADS : GEMM_THREADS_MMQ);
    cfg.dynamicSmemBytes = gemm_smem_bytes<TN, QT>();
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 1;
    at.val.clusterDim.y = 16;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kfn, &cfg) == cudaSuccess && n > 0) cached = 16;
  }
  cudaGetLastError();
  return cached;
}

template <int TN, int QT = QT_BF16>
int gemm_launch(const CUtensorMap& tmW, const CUtensorMap& tmX, __nv_bfloat16* Y, const float* bias, int N, int T, int K,
                int ldY, const GemmPlan& p, float* ws, int* counters, int epi_mode, const ArArgs& ar,
                cudaStream_t stream, const QwArgs& qw = QwArgs{nullptr, 0, nullptr, 0},
                const GroupArgs& gr = GroupArgs{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1}, int groups = 1,
                const RopeArgs& ro = RopeArgs{nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 0, 0, nullptr, nullptr},
                const NormArgs& nm = NormArgs{nullptr, 0.f, 0.f, nullptr, nullptr}) {
  using Cfg = GemmTile<TN>;
  static bool configured[64] = {false};  // per device ordinal: the attribute belongs to the device's copy of the kernel
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<TN, QT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         gemm_smem_bytes<TN, QT>());
    if (e != cudaSuccess) return (int)e;
    if (QT != QT_BF16) {
      // The packed-weight kernel moves registers between its warpgroups; the three budgets add up to what the launch
      // allocates only if the kernel was compiled for exactly MMQ_REGS_LAUNCH registers per thread.  A request for
      // more than the CTA owns would never be granted, so refuse to launch anything else.
      cudaFuncAttributes fa;
      e = cudaFuncGetAttributes(&fa, gemm_bf16_kernel<TN, QT>);
      if (e != cudaSuccess) return (int)e;
      if (fa.numRegs != MMQ_REGS_LAUNCH) return (int)cudaErrorInvalidConfiguration;
    }
    configured[dev] = true;
  }
  int splits = p.splits;
  if (p.cluster) {
    const int mc = gemm_max_cluster<TN, QT>();
    if (splits > mc) splits = mc;
  }
  dim3 grid(p.n_tiles, splits, gr.enabled ? (gr.row_offsets != nullptr ? groups * gr.t_tiles : groups) : p.t_tiles);
  const dim3 block(QT == QT_BF16 ? GEMM_THREADS : GEMM_THREADS_MMQ);
  cudaError_t le;
  GroupArgs grl = gr;
  grl.l2_prefetch_kb = g_oxb_gemm_l2_prefetch_kb;
  if (p.cluster && splits > 1) {
    le = oxb_launch_cluster(gemm_bf16_kernel<TN, QT>, grid, block, dim3(1, splits, 1), (size_t)gemm_smem_bytes<TN, QT>(), stream, tmW,
                            tmX, Y, bias, N, T, K, ldY, splits, ws, counters, epi_mode, ar, qw, grl, ro, nm);
  } else {
    le = oxb_launch(gemm_bf16_kernel<TN, QT>, grid, block, (size_t)gemm_smem_bytes<TN, QT>(), stream, tmW, tmX, Y, bias, N, T, K, ldY,
                    splits, ws, counters, epi_mode, ar, qw, grl, ro, nm);
  }
  if (le != cudaSuccess) return (int)le;
  OXB_CHECK_LAUNCH();
  return 0;
}

// dispatch on the token tile for a packed-weight format
template <int QT>
int gemm_launch_mmq(const CUtensorMap& tmX, __nv_bfloat16* Y, const float* bias, int N, int T, int K, int ldY,
                    const GemmPlan& p, float* ws, int* counters, int epi_mode, const ArArgs& ar, cudaStream_t stream,
                    const QwArgs& qw, const GroupArgs& gr = GroupArgs{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1}, int groups = 1,
                    const CUtensorMap* tmWq = nullptr) {
  // tmWq: byte map of the packed rows (needed by the staged Q4_K path); other formats never touch tmW
  const CUtensorMap& tmW = tmWq != nullptr ? *tmWq : tmX;
  switch (p.tn) {
    case 16: return gemm_launch<16, QT>(tmW, tmX, Y, bias, N, T, K, ldY, p, ws, counters, epi_mode, ar, stream, qw, gr, groups);
    case 32: return gemm_launch<32, QT>(tmW, tmX, Y, bias, N, T, K, ldY, p, ws, counters, epi_mode, ar, stream, qw, gr, groups);
    case 64: return gemm_launch<64, QT>(tmW, tmX, Y, bias, N, T, K, ldY, p, ws, counters, epi_mode, ar, stream, qw, gr, groups);
    case 128: return gemm_launch<128, QT>(tmW, tmX, Y, bias, N, T, K, ldY, p, ws, counters, epi_mode, ar, stream, qw, gr, groups);
    default: return (int)cudaErrorInvalidConfiguration;  // packed weights are planned with 128-token tiles at most
  }
}

}  // namespace oxb
