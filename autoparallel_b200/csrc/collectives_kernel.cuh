// Stand-alone all-gather and reduce-scatter over the same symmetric arena, signal pad and epoch
// protocol as the fused GEMM kernel (counterparts of _low_contention_all_gather /
// _low_contention_reduce_scatter, autoparallel/asynctp_ops.py:1524-1702). Plain 16-byte loads and
// stores, every peer addressed at once (piece q goes to / comes from peer rank+1+(q % (ws-1))).
// All waits are bounded like in the GEMM kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_kernel.cuh"

namespace apk {

struct CParams {
  int32_t ws, rank;
  uint32_t epoch;
  int32_t fp32;                          // reduce-scatter element type: 1 fp32, 0 bf16
  long long chunk_bytes;                 // one rank's part
  const uint8_t* src;                    // AG: local shard. RS: the full local input, ws chunks
  uint8_t* out;                          // AG: ws chunks. RS: one chunk
  uint8_t* symm_local;                   // this rank's arena half
  uint8_t* symm_peer[MAX_WORLD];
  uint32_t* flag_local;                  // AG: staged flags (FLAG_STRIDE apart). RS: per-source flags
  uint32_t* flag_peer[MAX_WORLD];
  int32_t flag_stride;                   // u32 words between two sources' flags
  uint32_t* ctrl;                        // zeroed per call
  float reduce_scale;
  uint32_t* status;
  long long timeout_cycles;
};

constexpr int COLL_THREADS = 512;

__device__ __forceinline__ bool coll_flag_wait(const uint32_t* flag, uint32_t target, const CParams& p, uint32_t code, uint32_t detail) {
  uint32_t spins = 0;
  long long t0 = 0;
  while (true) {
    const uint32_t v = ptx::ld_acquire_sys(flag);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++spins & 0x3fu) == 0) {
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > p.timeout_cycles) {
        atomicCAS(p.status, 0u, code | (detail << 8));
        return false;
      }
      __nanosleep(64);
    }
  }
}

// out[r] = shard of rank r. Each rank stages its shard in its arena half, releases the peers'
// "staged" flags, then pulls the peers' shards.
__global__ void __launch_bounds__(COLL_THREADS, 1) all_gather_kernel(const CParams p) {
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (COLL_THREADS / 32) + (threadIdx.x >> 5);
  const long long tw = (long long)gridDim.x * (COLL_THREADS / 32);
  const long long pieces = (p.chunk_bytes + PIECE_BYTES - 1) / PIECE_BYTES;
  uint8_t* own_out = p.out + (size_t)p.rank * p.chunk_bytes;
  for (long long q = gw; q < pieces; q += tw) {
    const long long off = q * PIECE_BYTES;
    const int n16 = (int)(min((long long)PIECE_BYTES, p.chunk_bytes - off) >> 4);
    copy_piece(p.src + off, own_out + off, p.ws > 1 ? p.symm_local + off : nullptr, n16, lane);
  }
  if (p.ws == 1) return;
  __threadfence_system();
  __syncwarp();
  if (lane == 0) {
    const uint32_t prev = atomicAdd(p.ctrl, 1u);
    if (prev == (uint32_t)tw - 1u) {
      __threadfence_system();
      for (int r = 0; r < p.ws; ++r) {
        if (r != p.rank) ptx::st_release_sys(p.flag_peer[r] + p.rank * p.flag_stride, p.epoch);
      }
    }
  }
  __syncwarp();
  const int npeers = p.ws - 1;
  uint32_t seen = 0;
  for (long long q = gw; q < pieces * npeers; q += tw) {
    const int src = (p.rank + 1 + (int)(q % npeers)) % p.ws;
    if (!(seen & (1u << src))) {
      bool ok = true;
      if (lane == 0) ok = coll_flag_wait(p.flag_local + src * p.flag_stride, p.epoch, p, ST_TIMEOUT_STAGED, (uint32_t)src);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) return;
      seen |= 1u << src;
    }
    const long long off = (q / npeers) * PIECE_BYTES;
    const int n16 = (int)(min((long long)PIECE_BYTES, p.chunk_bytes - off) >> 4);
    const uint8_t* peer = p.symm_peer[src];
    uint8_t* dst = p.out + (size_t)src * p.chunk_bytes;
    uint4 r[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = u * 32 + lane;
      if (i < n16) r[u] = ptx::ld_relaxed_sys_v4(peer + off + (size_t)i * 16);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = u * 32 + lane;
      if (i < n16) reinterpret_cast<uint4*>(dst + off)[i] = r[u];
    }
  }
}

// out = sum (or mean) over ranks of chunk `rank` of every rank's input. Each rank stores chunk d of
// its input into slot [rank] of peer d's arena half, releases peer d's flag for source `rank`
// once all of its CTAs are done, waits for the ws-1 flags addressed to it and adds the slots up.
__global__ void __launch_bounds__(COLL_THREADS, 1) reduce_scatter_kernel(const CParams p) {
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (COLL_THREADS / 32) + (threadIdx.x >> 5);
  const long long tw = (long long)gridDim.x * (COLL_THREADS / 32);
  const long long pieces = (p.chunk_bytes + PIECE_BYTES - 1) / PIECE_BYTES;
  const int npeers = p.ws - 1;
  if (p.ws > 1) {
    for (long long q = gw; q < pieces * npeers; q += tw) {
      const int dst = (p.rank + 1 + (int)(q % npeers)) % p.ws;
      const long long off = (q / npeers) * PIECE_BYTES;
      const int n16 = (int)(min((long long)PIECE_BYTES, p.chunk_bytes - off) >> 4);
      copy_piece(p.src + (size_t)dst * p.chunk_bytes + off, p.symm_peer[dst] + (size_t)p.rank * p.chunk_bytes + off, nullptr, n16, lane);
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(p.ctrl, 1u);
      if (prev == gridDim.x - 1u) {
        __threadfence_system();
        for (int r = 0; r < p.ws; ++r) {
          if (r != p.rank) ptx::st_release_sys(p.flag_peer[r] + p.rank * p.flag_stride, p.epoch);
        }
      }
      bool ok = true;
      for (int r = 0; r < p.ws && ok; ++r) {
        if (r != p.rank) ok = coll_flag_wait(p.flag_local + r * p.flag_stride, p.epoch, p, ST_TIMEOUT_PARTIAL, (uint32_t)r);
      }
      ok_s = ok ? 1 : 0;
    }
    __syncthreads();
    if (!ok_s) return;
  }
  const uint8_t* mine = p.src + (size_t)p.rank * p.chunk_bytes;
  const long long n16_total = p.chunk_bytes >> 4;
  for (long long i = (long long)blockIdx.x * COLL_THREADS + threadIdx.x; i < n16_total; i += (long long)gridDim.x * COLL_THREADS) {
    const uint4 own = __ldcg(reinterpret_cast<const uint4*>(mine) + i);
    if (p.fp32) {
      float4 acc = *reinterpret_cast<const float4*>(&own);
      for (int r = 0; r < p.ws; ++r) {
        if (r == p.rank) continue;
        const uint4 qv = ptx::ld_cg_v4(p.symm_local + (size_t)r * p.chunk_bytes + (size_t)i * 16);
        const float4 q = *reinterpret_cast<const float4*>(&qv);
        acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
      }
      acc.x *= p.reduce_scale; acc.y *= p.reduce_scale; acc.z *= p.reduce_scale; acc.w *= p.reduce_scale;
      reinterpret_cast<float4*>(p.out)[i] = acc;
    } else {
      float acc[8];
      const uint32_t w0[4] = {own.x, own.y, own.z, own.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] = __uint_as_float(w0[e] << 16);
        acc[2 * e + 1] = __uint_as_float(w0[e] & 0xffff0000u);
      }
      for (int r = 0; r < p.ws; ++r) {
        if (r == p.rank) continue;
        const uint4 q = ptx::ld_cg_v4(p.symm_local + (size_t)r * p.chunk_bytes + (size_t)i * 16);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] += __uint_as_float(w[e] << 16);
          acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
        }
      }
      uint4 o;
      o.x = pack_bf16(acc[0] * p.reduce_scale, acc[1] * p.reduce_scale);
      o.y = pack_bf16(acc[2] * p.reduce_scale, acc[3] * p.reduce_scale);
      o.z = pack_bf16(acc[4] * p.reduce_scale, acc[5] * p.reduce_scale);
      o.w = pack_bf16(acc[6] * p.reduce_scale, acc[7] * p.reduce_scale);
      reinterpret_cast<uint4*>(p.out)[i] = o;
    }
  }
}

}  // namespace apk
