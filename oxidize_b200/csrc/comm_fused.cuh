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
  int mode;                           // 0 = one-shot (push to all), 1 = two-shot (reduce at an owner, broadcast)
  int t_max, n_max, max_tiles;        // receive buffer geometry
  unsigned long long timeout_ns;      // bound on the peer-flag wait
  __nv_bfloat16* data[AR_MAX_WORLD];  // peers' receive buffers [2][world + 1][t_max][n_max] (slot `world` = results)
  uint32_t* flags[AR_MAX_WORLD];      // peers' flag arrays     [2][world + 1][max_tiles]
  int* ctrl;                          // local: [0] call counter, [1] CTAs done
  const __nv_bfloat16* residual;      // optional: added to the reduced sum (local, [T, ldY])
};

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
  __threadfence_system();
  asm volatile("bar.sync 1, 128;" ::: "memory");
  // ---- signal: one thread per destination
  if (tid < W) st_release_sys(ar.flags[tid] + ((size_t)parity * (W + 1) + ar.rank) * ar.max_tiles + tile_id, 1u);
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
  if (*abort_flag) return false;
  // ---- reduce the W partials in rank order (L2 loads: the lines were written by peers)
  const __nv_bfloat16* mine = ar.data[ar.rank] + (size_t)parity * (W + 1) * slot_elems;
  if (col_ok) {
    for (int t = trow; t < tmax; t += 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = bias_v;
      for (int s = 0; s < W; ++s) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mine + (size_t)s * slot_elems +
                                                              (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8));
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      __nv_bfloat16* out = Y + (size_t)(t0 + t) * ldY + n0 + chunk * 8;
      if (ar.residual != nullptr) {
        const uint4 rv = *reinterpret_cast<const uint4*>(ar.residual + (size_t)(t0 + t) * ldY + n0 + chunk * 8);
        const uint32_t u[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out) = o;
    }
  }
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

// Two-shot variant for larger rank counts: the piece (tile_id) is reduced at ONE owner rank
// (tile_id mod world) and the result broadcast, so each rank moves 2·(W-1)/W of the tensor over
// NVLink instead of (W-1)×.  Steps for the 128 epilogue threads of the CTA holding piece `tile_id`:
//   1. push the partial piece into the owner's slot [rank]; raise the owner's arrival flag;
//   2. owner only: wait for all W arrivals, sum in rank order, push the sum into every rank's result
//      slot, raise every rank's result flag;
//   3. wait for the result flag, copy the piece (+ residual) into Y.
// `stage` is overwritten by the owner with the reduced piece.
__device__ __forceinline__ bool ar_exchange_tile_twoshot(const ArArgs& ar, uint8_t* stage, int parity, int tile_id, int n0,
                                                         int t0, int tmax, int N, __nv_bfloat16* Y, int ldY,
                                                         volatile int* abort_flag, int tid) {
  const int W = ar.world;
  const int owner = tile_id % W;
  const int chunk = tid & 15, trow = tid >> 4;
  const bool col_ok = n0 + chunk * 8 < N;
  const size_t slot_elems = (size_t)ar.t_max * ar.n_max;
  const size_t pbase = (size_t)parity * (W + 1);
  // ---- 1. partial -> owner
  {
    __nv_bfloat16* dst = ar.data[owner] + (pbase + ar.rank) * slot_elems;
    if (col_ok)
      for (int t = trow; t < tmax; t += 8)
        *reinterpret_cast<uint4*>(dst + (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8) =
            *reinterpret_cast<const uint4*>(stage + t * 256 + chunk * 16);
  }
  __threadfence_system();
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (tid == 0) st_release_sys(ar.flags[owner] + (pbase + ar.rank) * ar.max_tiles + tile_id, 1u);
  // ---- 2. owner reduces and broadcasts
  if (owner == ar.rank) {
    if (tid < W) ar_wait_flag(ar.flags[ar.rank] + (pbase + tid) * ar.max_tiles + tile_id, ar.timeout_ns, abort_flag, tid);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!*abort_flag) {
      const __nv_bfloat16* mine = ar.data[ar.rank] + pbase * slot_elems;
      if (col_ok) {
        for (int t = trow; t < tmax; t += 8) {
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          for (int s = 0; s < W; ++s) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mine + (size_t)s * slot_elems +
                                                                  (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(u[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]);
          o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]);
          o.w = pack_bf16x2(acc[6], acc[7]);
          for (int k = 1; k <= W; ++k) {
            const int d = (ar.rank + k) % W;
            *reinterpret_cast<uint4*>(ar.data[d] + (pbase + W) * slot_elems + (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8) = o;
          }
        }
      }
      __threadfence_system();
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!*abort_flag && tid < W) st_release_sys(ar.flags[tid] + (pbase + W) * ar.max_tiles + tile_id, 1u);
  }
  // ---- 3. result -> Y
  if (tid == 0) ar_wait_flag(ar.flags[ar.rank] + (pbase + W) * ar.max_tiles + tile_id, ar.timeout_ns, abort_flag, W);
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (*abort_flag) return false;
  const __nv_bfloat16* res = ar.data[ar.rank] + (pbase + W) * slot_elems;
  if (col_ok) {
    for (int t = trow; t < tmax; t += 8) {
      uint4 v = __ldcg(reinterpret_cast<const uint4*>(res + (size_t)(t0 + t) * ar.n_max + n0 + chunk * 8));
      if (ar.residual != nullptr) {
        const uint4 rv = *reinterpret_cast<const uint4*>(ar.residual + (size_t)(t0 + t) * ldY + n0 + chunk * 8);
        uint32_t a[4] = {v.x, v.y, v.z, v.w};
        const uint32_t b[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = unpack_bf16x2(a[j]), fb = unpack_bf16x2(b[j]);
          a[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
        }
        v = make_uint4(a[0], a[1], a[2], a[3]);
      }
      *reinterpret_cast<uint4*>(Y + (size_t)(t0 + t) * ldY + n0 + chunk * 8) = v;
    }
  }
  return true;
}

// picks the exchange by ar.mode
__device__ __forceinline__ bool ar_exchange(const ArArgs& ar, uint8_t* stage, int parity, int tile_id, int n0, int t0,
                                            int tmax, int N, __nv_bfloat16* Y, int ldY, volatile int* abort_flag, int tid) {
  if (ar.mode == 1) return ar_exchange_tile_twoshot(ar, stage, parity, tile_id, n0, t0, tmax, N, Y, ldY, abort_flag, tid);
  return ar_exchange_tile(ar, stage, parity, tile_id, n0, t0, tmax, N, Y, ldY, 0.f, abort_flag, tid);
}

// Stand-alone one-shot all-reduce of a [T, N] bf16 tensor through the same buffers (used for
// tensors that do not come out of a GEMM, e.g. the MoE combine): grid = N/128 tiles.
__global__ void __launch_bounds__(128)
allreduce_oneshot_kernel(const ArArgs ar, const __nv_bfloat16* __restrict__ X, __nv_bfloat16* __restrict__ Y, int T, int N,
                         int ld) {
  extern __shared__ __align__(16) uint8_t ar_stage[];  // [T][256] bytes
  __shared__ int s_parity, s_abort;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * 128;
  if (tid == 0) {
    s_parity = ar.ctrl[0] & 1;
    s_abort = 0;
  }
  const int chunk = tid & 15, trow = tid >> 4;
  for (int t = trow; t < T; t += 8) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n0 + chunk * 8 < N) v = *reinterpret_cast<const uint4*>(X + (size_t)t * ld + n0 + chunk * 8);
    *reinterpret_cast<uint4*>(ar_stage + t * 256 + chunk * 16) = v;
  }
  __syncthreads();
  ar_exchange(ar, ar_stage, s_parity, blockIdx.x, n0, 0, T, N, Y, ld, &s_abort, tid);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int done = atomicAdd(&ar.ctrl[1], 1);
    if (done == (int)gridDim.x - 1) {
      ar.ctrl[1] = 0;
      __threadfence();
      ar.ctrl[0] = ar.ctrl[0] + 1;
    }
  }
}

}  // namespace oxb
