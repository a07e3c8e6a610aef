// In-kernel collectives over NVLink peer memory, fused into the GEMM epilogue.
//
// One-shot all-reduce of a row-parallel GEMM (attn_output, ffn_down): as soon as a CTA has its
// 128-row × T-token partial tile it pushes the tile (bf16) straight into every peer's symmetric
// receive buffer with 16-byte P2P stores, raises a per-(source, tile) flag with a system-scope
// release store, then waits (bounded) for the same tile from every peer and reduces the W
// partials in fixed rank order — so every rank obtains bit-identical sums, tile by tile, while
// other CTAs are still in their MMA main loop.  There is no separate collective launch and no
// host involvement; the reference has nothing comparable (its only collectives are a TCP ring,
// oxidize-core/src/mesh/ring.rs:245-365).
//
// Buffers alternate between two parities per call so that a fast peer, which can be at most
// one call ahead, never overwrites data or flags that are still being read; the parity comes
// from a device-side call counter, which keeps CUDA-graph replays consistent across ranks.
// Plain peer loads/stores only: no multimem and no cluster-scope TMA here.
#pragma once
#include "common.cuh"

namespace oxb {

constexpr int AR_MAX_WORLD = 8;

struct ArArgs {
  int world;                          // 0 = no collective
  int rank;
  int mode;                           // 0 = one-shot push with per-piece flags, 1 = two-shot with in-data flags (LL)
  int t_max, n_max, max_tiles;        // receive buffer geometry
  unsigned long long timeout_ns;      // bound on the peer-flag wait
  __nv_bfloat16* data[AR_MAX_WORLD];  // peers' receive buffers: [2][world + 1][t_max][n_max] x 4 bytes (LL wire format;
                                      // the one-shot exchange uses the first half as bf16; slot `world` = results)
  uint32_t* flags[AR_MAX_WORLD];      // peers' flag arrays     [2][world + 1][max_tiles]
  int* ctrl;                          // local: [0] call counter, [1] CTAs done
  const __nv_bfloat16* residual;      // optional: added to the reduced sum (local, [T, ldY])
  unsigned long long* trace;          // optional: phase timestamps (globaltimer ns) of piece 0, for latency analysis
};

#define AR_STAMP(i)                                                                  \
  do {                                                                               \
    if (ar.trace != nullptr && tile_id == 0 && tid == 0) ar.trace[i] = globaltimer_ns(); \
  } while (0)

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Sum of the W partial copies of one 16-byte chunk for two token rows at once: the 2*W loads are
// issued before any add so that their latencies overlap; the adds run in rank order (reproducible).
__device__ __forceinline__ void ar_sum2(const __nv_bfloat16* p0, const __nv_bfloat16* p1, bool has1, size_t slot_elems, int W,
                                        float (&a0)[8], float (&a1)[8]) {
  uint4 v0[AR_MAX_WORLD], v1[AR_MAX_WORLD];
#pragma unroll
  for (int s = 0; s < AR_MAX_WORLD; ++s) {
    v0[s] = make_uint4(0, 0, 0, 0);
    v1[s] = make_uint4(0, 0, 0, 0);
    if (s < W) {
      v0[s] = __ldcg(reinterpret_cast<const uint4*>(p0 + (size_t)s * slot_elems));
      if (has1) v1[s] = __ldcg(reinterpret_cast<const uint4*>(p1 + (size_t)s * slot_elems));
    }
  }
#pragma unroll
  for (int s = 0; s < AR_MAX_WORLD; ++s) {
    if (s < W) {
      const uint32_t u0[4] = {v0[s].x, v0[s].y, v0[s].z, v0[s].w};
      const uint32_t u1[4] = {v1[s].x, v1[s].y, v1[s].z, v1[s].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f0 = unpack_bf16x2(u0[j]), f1 = unpack_bf16x2(u1[j]);
        a0[2 * j] += f0.x;
        a0[2 * j + 1] += f0.y;
        a1[2 * j] += f1.x;
        a1[2 * j + 1] += f1.y;
      }
    }
  }
}

__device__ __forceinline__ uint4 ar_pack8(const float (&a)[8]) {
  return make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
}

__device__ __forceinline__ void ar_add8(float (&a)[8], const uint4 v) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(u[j]);
    a[2 * j] += f.x;
    a[2 * j + 1] += f.y;
  }
}

// Executed by the 128 epilogue threads (tid 0..127) of the CTA that holds the finished partial
// tile in shared memory as bf16 [tn][128] (`stage`).  Pushes, signals, waits, reduces and
// writes Y.  Returns false if the peer wait timed out (status word set, nothing written).
__device__ __forceinline__ bool ar_exchange_tile(const ArArgs& ar, const uint8_t* stage, int parity, int tile_id,
                                                 int n0, int t0, int tmax, int N, __nv_bfloat16* Y, int ldY,
                                                 const float bias_v, volatile int* abort_flag, int tid) {
  const int W = ar.world;
  const int chunk = tid & 15;     // 16-byte chunk inside the 256-byte tile row
  const int trow = tid >> 4;      // 8 tokens per pass
  const bool col_ok = n0 + chunk * 8 < N;
  const size_t slot_elems = (size_t)ar.t_max * ar.n_max;
  AR_STAMP(0);
  // ---- push my partial to every rank (self last)
  for (int k = 1; k <= W; ++k) {
    const int d = (ar.rank + k) % W;
    __nv_bfloat16* dst = ar.data[d] + ((size_t)parity * (W + 1) + ar.rank) * slot_elems;
    if (col_ok) {
      for (int t = trow; t < tmax; t += 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(stage + t * 256 + chunk * 16);
        *reinterpret_cast<uint4*>(dst + (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8) = v;
      }
    }
  }
  AR_STAMP(1);
  // The CTA barrier orders every thread's stores before the releasing threads; their system-scope
  // release stores are cumulative, so no per-thread fence is needed (it would cost one more NVLink
  // round trip).
  asm volatile("bar.sync 1, 128;" ::: "memory");
  AR_STAMP(2);
  // ---- signal: one thread per destination
  if (tid < W) st_release_sys(ar.flags[tid] + ((size_t)parity * (W + 1) + ar.rank) * ar.max_tiles + tile_id, 1u);
  AR_STAMP(3);
  // ---- wait for every source's copy of this tile (bounded)
  if (tid < W) {
    uint32_t* f = ar.flags[ar.rank] + ((size_t)parity * (W + 1) + tid) * ar.max_tiles + tile_id;
    const unsigned long long t_start = globaltimer_ns();
    bool got = false;
    for (unsigned it = 0;; ++it) {
      if (ld_acquire_sys(f) != 0u) {
        got = true;
        break;
      }
      if (*abort_flag) break;
      if ((it & 63) == 63 && globaltimer_ns() - t_start > ar.timeout_ns) break;
    }
    if (got) {
      *f = 0u;  // consumed; the next writer of this flag is two calls away
    } else if (!*abort_flag) {
      *abort_flag = 1;
      oxb_report(OXB_TIMEOUT_PEER_FLAG, tid);
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  AR_STAMP(4);
  if (*abort_flag) return false;
  // ---- reduce the W partials in rank order (L2 loads: the lines were written by peers)
  const __nv_bfloat16* mine = ar.data[ar.rank] + (size_t)parity * (W + 1) * slot_elems;
  if (col_ok) {
    for (int t = trow; t < tmax; t += 16) {
      const bool has1 = t + 8 < tmax;
      float a0[8], a1[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a0[j] = a1[j] = bias_v;
      const size_t off0 = (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8;
      uint4 r0 = make_uint4(0, 0, 0, 0), r1 = r0;
      if (ar.residual != nullptr) {
        r0 = *reinterpret_cast<const uint4*>(ar.residual + (size_t)(t0 + t) * ldY + n0 + chunk * 8);
        if (has1) r1 = *reinterpret_cast<const uint4*>(ar.residual + (size_t)(t0 + t + 8) * ldY + n0 + chunk * 8);
      }
      ar_sum2(mine + off0, mine + off0 + (size_t)8 * ar.n_max, has1, slot_elems, W, a0, a1);
      if (ar.residual != nullptr) {
        ar_add8(a0, r0);
        ar_add8(a1, r1);
      }
      *reinterpret_cast<uint4*>(Y + (size_t)(t0 + t) * ldY + n0 + chunk * 8) = ar_pack8(a0);
      if (has1) *reinterpret_cast<uint4*>(Y + (size_t)(t0 + t + 8) * ldY + n0 + chunk * 8) = ar_pack8(a1);
    }
  }
  AR_STAMP(5);
  return true;
}

// Bounded wait on one local flag word; consumes it (resets to 0) on success.
__device__ __forceinline__ bool ar_wait_flag(uint32_t* f, unsigned long long timeout_ns, volatile int* abort_flag, int detail) {
  const unsigned long long t_start = globaltimer_ns();
  for (unsigned it = 0;; ++it) {
    if (ld_acquire_sys(f) != 0u) {
      *f = 0u;
      return true;
    }
    if (*abort_flag) return false;
    if ((it & 63) == 63 && globaltimer_ns() - t_start > timeout_ns) break;
  }
  if (!*abort_flag) {
    *abort_flag = 1;
    oxb_report(OXB_TIMEOUT_PEER_FLAG, detail);
  }
  return false;
}

// ---- "LL" exchange: reduce-scatter + all-gather with the flag inside the data.
// Every 8 bytes on the wire are {4 bytes payload, 4 bytes epoch}; an aligned 8-byte store is atomic, so a
// receiver that sees the epoch of THIS call in a word also sees its payload: no fence, no separate flag,
// no flag reset, and the latency of a hop is one NVLink traversal instead of a round trip plus one.  The
// price is 2x bytes on the wire, which the two-shot shape more than pays for: each rank moves
// 2*(W-1)/W of the tensor (x2) instead of (W-1)x.
// The piece is cut into 16-byte chunks q (token q/16, 8 columns q%16); token t of the piece is reduced
// by rank t mod W, so a warp's stores to one destination stay contiguous (256-byte rows: scattering
// single chunks over the ranks gave NVLink packets of 32 bytes and a third of the throughput).
// For the 128 epilogue threads of the CTA that holds the piece:
//   1. chunk q = tid + 128 i goes to rank ((q / 16) mod W), slot [this rank];
//   2. the chunks of the tokens owned by this rank are polled from all W slots, summed in rank order
//      (bit-identical everywhere) and the sum is written to every rank's result slot;
//   3. chunk q = tid + 128 i is polled from the result slot and written to Y (+ residual).
// The CTAs with the same piece index on the W ranks thus form one team; all of them do equal work.
// Buffers alternate between two parities per call (a rank can be at most one call ahead of another).
__device__ __forceinline__ void ll_store32(uint8_t* dst, const uint4 v, uint32_t e) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(e), "r"(v.y), "r"(e) : "memory");
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 16), "r"(v.z), "r"(e), "r"(v.w), "r"(e)
               : "memory");
}
__device__ __forceinline__ bool ll_try_load32(const uint8_t* src, uint32_t e, uint4& out) {
  uint32_t a0, f0, a1, f1, a2, f2, a3, f3;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(f0), "=r"(a1), "=r"(f1) : "l"(src) : "memory");
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(a2), "=r"(f2), "=r"(a3), "=r"(f3)
               : "l"(src + 16)
               : "memory");
  out = make_uint4(a0, a1, a2, a3);
  return f0 == e && f1 == e && f2 == e && f3 == e;
}

__device__ __forceinline__ bool ar_exchange_ll(const ArArgs& ar, const uint8_t* stage, uint32_t call, int tile_id, int n0,
                                               int t0, int tmax, int N, __nv_bfloat16* Y, int ldY, volatile int* abort_flag,
                                               int tid, unsigned long long* ssq_out = nullptr) {
  const int W = ar.world;
  const uint32_t epoch = (call + 1u) != 0u ? call + 1u : 1u;
  const size_t slot_bytes = (size_t)ar.t_max * ar.n_max * 4;  // 4 bytes per bf16 element on the wire
  const size_t pbase = (size_t)(call & 1u) * (W + 1);
  const int Q = tmax * 16;
  AR_STAMP(0);
  // ---- 1. scatter the partial chunks to their owners
  for (int q = tid; q < Q; q += 128) {
    const int t = q >> 4, c = q & 15;
    if (n0 + c * 8 >= N) continue;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + t * 256 + c * 16);
    uint8_t* dst = reinterpret_cast<uint8_t*>(ar.data[t % W]) + (pbase + ar.rank) * slot_bytes +
                   ((size_t)(t0 + t) * ar.n_max + n0 + c * 8) * 4;
    ll_store32(dst, v, epoch);
  }
  AR_STAMP(1);
  const uint8_t* mine = reinterpret_cast<const uint8_t*>(ar.data[ar.rank]) + pbase * slot_bytes;
  const unsigned long long t_start = globaltimer_ns();
  bool fail = false;
  // ---- 2. reduce the chunks this rank owns, broadcast the sums
  for (int j = tid; !fail; j += 128) {
    const int t = (j >> 4) * W + ar.rank, c = j & 15;  // j-th chunk of the tokens this rank owns
    if (t >= tmax) break;
    if (n0 + c * 8 >= N) continue;
    const size_t off = ((size_t)(t0 + t) * ar.n_max + n0 + c * 8) * 4;
    uint4 v[AR_MAX_WORLD];
    unsigned pending = (1u << W) - 1u;
    for (unsigned it = 0; pending != 0u; ++it) {
#pragma unroll
      for (int s = 0; s < AR_MAX_WORLD; ++s)
        if (s < W && ((pending >> s) & 1u) && ll_try_load32(mine + (size_t)s * slot_bytes + off, epoch, v[s])) pending &= ~(1u << s);
      if (pending != 0u && (*abort_flag || ((it & 15u) == 15u && globaltimer_ns() - t_start > ar.timeout_ns))) {
        fail = true;
        break;
      }
    }
    if (fail) break;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int s = 0; s < AR_MAX_WORLD; ++s)
      if (s < W) ar_add8(acc, v[s]);
    const uint4 o = ar_pack8(acc);
    for (int k = 1; k <= W; ++k)
      ll_store32(reinterpret_cast<uint8_t*>(ar.data[(ar.rank + k) % W]) + (pbase + W) * slot_bytes + off, o, epoch);
  }
  AR_STAMP(2);
  // ---- 3. gather the reduced piece
  // (the 16 lanes that hold one token row take every branch below together: the verdict of a failed poll
  // is shared inside that half warp, so the row's sum of squares can be formed with shuffles)
  const unsigned hmask = (tid & 16) ? 0xFFFF0000u : 0x0000FFFFu;
  const uint8_t* res = mine + (size_t)W * slot_bytes;
  fail = __any_sync(hmask, fail);
  for (int q0 = tid; q0 < Q && !fail; q0 += 128 * 4) {
    uint4 v[4];
    unsigned pending = 0u;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int q = q0 + 128 * u;
      if (q < Q && n0 + (q & 15) * 8 < N) pending |= 1u << u;
    }
    const unsigned valid = pending;
    // the residual rows are local: their reads are issued before the poll, whose wait hides them
    uint4 resid[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int q = q0 + 128 * u;
      resid[u] = make_uint4(0, 0, 0, 0);
      if (ar.residual != nullptr && ((valid >> u) & 1u))
        resid[u] = *reinterpret_cast<const uint4*>(ar.residual + (size_t)(t0 + (q >> 4)) * ldY + n0 + (q & 15) * 8);
    }
    for (unsigned it = 0; pending != 0u; ++it) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + 128 * u;
        if (((pending >> u) & 1u) &&
            ll_try_load32(res + ((size_t)(t0 + (q >> 4)) * ar.n_max + n0 + (q & 15) * 8) * 4, epoch, v[u]))
          pending &= ~(1u << u);
      }
      if (pending != 0u && (*abort_flag || ((it & 15u) == 15u && globaltimer_ns() - t_start > ar.timeout_ns))) {
        fail = true;
        break;
      }
    }
    fail = __any_sync(hmask, fail);
    if (fail) break;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int q = q0 + 128 * u;
      float ss = 0.f;
      if ((valid >> u) & 1u) {
        const size_t yo = (size_t)(t0 + (q >> 4)) * ldY + n0 + (q & 15) * 8;
        uint4 o = v[u];
        if (ar.residual != nullptr) {
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
          ar_add8(acc, o);
          ar_add8(acc, resid[u]);
          o = ar_pack8(acc);
        }
        *reinterpret_cast<uint4*>(Y + yo) = o;
        if (ssq_out != nullptr) {
          const uint32_t w4[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = unpack_bf16x2(w4[i]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
      if (ssq_out != nullptr && q < Q) {  // q < Q holds for all 16 lanes of the row or for none
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(hmask, ss, o2);
        if ((q & 15) == 0) {  // fixed-point add: the total does not depend on the order of the tiles (NormArgs)
          ss = fminf(ss, 3.0e10f);
          atomicAdd(ssq_out + (size_t)(t0 + (q >> 4)) * 16 /*SUMSQ_STRIDE*/, (unsigned long long)(ss * 268435456.f + 0.5f));
        }
      }
    }
  }
  AR_STAMP(3);
  if (fail && !*abort_flag) {
    *abort_flag = 1;
    oxb_report(OXB_TIMEOUT_PEER_FLAG, tile_id);
  }
  return !fail;
}

// picks the exchange by ar.mode; `call` is the device-side call counter of this collective
__device__ __forceinline__ bool ar_exchange(const ArArgs& ar, const uint8_t* stage, int call, int tile_id, int n0, int t0,
                                            int tmax, int N, __nv_bfloat16* Y, int ldY, volatile int* abort_flag, int tid,
                                            unsigned long long* ssq_out = nullptr) {
  // (the per-row sums of squares exist on the two-shot exchange only; the host does not ask for them otherwise)
  if (ar.mode == 1) return ar_exchange_ll(ar, stage, (uint32_t)call, tile_id, n0, t0, tmax, N, Y, ldY, abort_flag, tid, ssq_out);
  return ar_exchange_tile(ar, stage, call & 1, tile_id, n0, t0, tmax, N, Y, ldY, 0.f, abort_flag, tid);
}

// Host side: fill the kernel argument block of one collective call from the symmetric-buffer pointers.
inline int fill_ar(ArArgs& ar, int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl,
                   int t_max, int n_max, int max_tiles, unsigned long long timeout_ns, const void* residual) {
  memset(&ar, 0, sizeof(ar));
  ar.mode = world >= g_oxb_ar_ll_min_world ? 1 : 0;
  ar.trace = g_oxb_ar_trace;
  if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world || ctrl == nullptr) return (int)cudaErrorInvalidValue;
  ar.world = world;
  ar.rank = rank;
  ar.t_max = t_max;
  ar.n_max = n_max;
  ar.max_tiles = max_tiles;
  ar.timeout_ns = timeout_ns;
  ar.ctrl = ctrl;
  ar.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  for (int i = 0; i < world; ++i) {
    ar.data[i] = reinterpret_cast<__nv_bfloat16*>(data_ptrs[i]);
    ar.flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  return 0;
}

// Stand-alone one-shot all-reduce of a [T, N] bf16 tensor through the same buffers (used for
// tensors that do not come out of a GEMM, e.g. the MoE combine): grid = N/128 tiles.
static __global__ void __launch_bounds__(128)
allreduce_oneshot_kernel(const ArArgs ar, const __nv_bfloat16* __restrict__ X, __nv_bfloat16* __restrict__ Y, int T, int N,
                         int ld, int tg) {
  extern __shared__ __align__(16) uint8_t ar_stage[];  // [tg][256] bytes
  __shared__ int s_call, s_abort;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * 128;
  const int t0 = blockIdx.y * tg;
  const int tmax = min(tg, T - t0);
  const int piece = blockIdx.y * gridDim.x + blockIdx.x;
  if (ar.trace != nullptr && piece == 0 && tid == 0) ar.trace[9] = globaltimer_ns();
  if (tid == 0) {
    s_call = ar.ctrl[0];
    s_abort = 0;
  }
  const int chunk = tid & 15, trow = tid >> 4;
  for (int t = trow; t < tmax; t += 8) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n0 + chunk * 8 < N) v = *reinterpret_cast<const uint4*>(X + (size_t)(t0 + t) * ld + n0 + chunk * 8);
    *reinterpret_cast<uint4*>(ar_stage + t * 256 + chunk * 16) = v;
  }
  __syncthreads();
  ar_exchange(ar, ar_stage, s_call, piece, n0, t0, tmax, N, Y, ld, &s_abort, tid);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int done = atomicAdd(&ar.ctrl[1], 1);
    if (done == (int)(gridDim.x * gridDim.y) - 1) {
      ar.ctrl[1] = 0;
      __threadfence();
      ar.ctrl[0] = ar.ctrl[0] + 1;
      if (ar.trace != nullptr) ar.trace[10] = globaltimer_ns();  // last CTA of the grid leaves
    }
  }
}

}  // namespace oxb
