// Persistent tcgen05/TMEM GEMM for sm_100a with the two async-TP fusions built in.
//
// One CTA per SM, 12 warps:
//   warp 0      TMA producer: waits for the rows of A it needs to be present in local
//               memory (all-gather mode), then streams A/B tiles into a shared-memory ring.
//   warp 1      MMA issuer: one thread issues tcgen05.mma into a double-buffered TMEM
//               accumulator (2 x BN fp32 columns).
//   warps 2-5   epilogue: tcgen05.ld -> scale/bias/convert -> swizzled shared-memory staging -> TMA
//               store. In reduce-scatter mode a tile owned by another rank leaves as linear 4 KiB
//               bulk copies into that rank's arena over NVLink and its per-tile flag is released
//               (several tiles in flight, flags in pairs behind one system fence); tiles owned by
//               this rank are computed last and summed with the partials that arrived.
//   warps 6-11  communication (all-gather mode): stage the local shard in the symmetric
//               buffer, tell the peers, then pull the peers' shards into the local gathered-A
//               buffer in 4 KiB pieces, bumping a per-row-block counter the producer waits on.
//
// Like the reference's pipelines the local rank's rows are consumed first by the all-gather
// (autoparallel/asynctp_ops.py:153) and produced last by the reduce-scatter (:321). Unlike them
// (one peer per step, :155-164, :250-315) the peers' rows are interleaved row block by row block
// so that a GPU exchanges data with all of its peers at once (see decode_tile).
//
// Every wait (mbarrier, flag, counter) is bounded by a cycle budget; when it runs out the
// kernel records a code in the status word, raises a CTA-wide abort flag, drains its own
// copies, frees TMEM and returns.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace apk {

constexpr int BM = 128;             // rows per tile = TMEM lanes
constexpr int ROW_BYTES = 128;      // bytes per shared-memory row = TMA inner box = swizzle span
constexpr int MAX_B = 4;            // weight matrices sharing one gathered A
constexpr int MAX_WORLD = 8;
constexpr int EPI_WARPS = 4;
constexpr int COMM_WARPS = 6;
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS + COMM_WARPS);
constexpr int PIECE_BYTES = 4096;   // unit of the all-gather pull: 32 lanes x 16 B x 8
constexpr int RS_LAG = 4;          // reduce-scatter: default distance (row blocks) between the peers' row block j and the own one
constexpr int FLAG_STRIDE = 32;     // u32 words between two ranks' "staged" flags (128 B)

enum Mode : int32_t { MODE_PLAIN = 0, MODE_AG = 1, MODE_RS = 2 };

// Status codes written (first one wins) to the status word when a wait gives up.
enum Status : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT_MBAR = 1,       // a pipeline mbarrier never completed
  ST_TIMEOUT_STAGED = 2,     // a peer never announced its staged shard
  ST_TIMEOUT_READY = 3,      // rows of a gathered chunk never arrived locally
  ST_TIMEOUT_PARTIAL = 4,    // a peer's reduce-scatter partial never arrived
};

struct alignas(64) KParams {
  CUtensorMap tmA0;            // plain / RS: all of A. AG: the local shard [rows_per_rank, K]
  CUtensorMap tmA1;            // AG: the gathered A [M, K]
  CUtensorMap tmB[MAX_B];
  CUtensorMap tmBp[MAX_B];             // CTA pairs, K-contiguous B: box of BN/2 rows (each CTA loads half of N)
  CUtensorMap tmOut[MAX_B];            // bf16 outputs, box 32 rows x 64 columns (TMA stores)
  int32_t mode, ws, rank, nB;
  int32_t M, K, rows_per_rank, elem_bytes;
  int32_t ag_ksplit;           // AG along the LAST dim: shards are K-slices [rows, K]; out = sum_r A_r @ B[r*K:(r+1)*K]
  int32_t rs_colsplit;         // RS along the LAST dim: rank d receives columns [d*N, (d+1)*N) of all rows
  int32_t N[MAX_B];
  int32_t b_nmajor[MAX_B];     // 1: B is [K][N] with N contiguous; 0: K contiguous
  void* out[MAX_B];
  int64_t ldo[MAX_B];
  int32_t out_fp32[MAX_B];
  int32_t out_f16[MAX_B];      // 16-bit outputs are IEEE half instead of bf16
  int32_t in_f16;              // A and B are IEEE half instead of bf16 (kind::f16 takes either)
  int32_t out_tma[MAX_B];      // tmOut[b] is valid
  // ---- scaled (fp8) epilogue
  int32_t a_scale_mode;        // 0 none, 1 one scalar, 2 one per row
  const float* a_scale_own;    // AG row-wise-sharded: scales of the local shard's rows
  const float* a_scale_full;   // scalar, or per-row indexed by the global row
  const float* b_scale[MAX_B];
  int32_t b_scale_mode[MAX_B]; // 0 none, 1 scalar, 2 per column
  const void* bias[MAX_B];     // per column, nullable
  int32_t bias_fp32[MAX_B];
  const float* result_scale[MAX_B];
  // ---- all-gather
  const uint8_t* ag_src;               // local shard bytes
  uint8_t* ag_symm_local;              // this rank's symmetric staging buffer (current parity)
  const uint8_t* ag_symm_peer[MAX_WORLD];
  uint8_t* ag_gathered;                // [M, K]
  int32_t ag_copy_own;                 // also place the local shard in ag_gathered
  int32_t ag_has_scale;
  int64_t ag_chunk_bytes;              // rows_per_rank * K * elem_bytes
  int64_t ag_scale_off;                // offset of the row scales inside the symmetric buffer
  const float* ag_scale_src;
  float* ag_scale_gathered;            // [M]
  uint32_t* staged_local;              // [ws * FLAG_STRIDE] in this rank's signal pad
  uint32_t* staged_peer[MAX_WORLD];
  uint32_t* ready;                     // [ws * tiles_m_per_chunk] local counters, zeroed per call
  uint32_t* ctrl;                      // local scratch counters, zeroed per call
  // ---- reduce-scatter
  uint8_t* rs_arena_local;             // partials (current parity): bf16 blocked [ws][tile][BN/64][4][32][64],
                                       // fp32 row-major [ws][rs_slot_rows][N]
  uint8_t* rs_arena_peer[MAX_WORLD];
  float* rs_sum_local;                 // bf16 partials: [tile][BN/64][4] blocks of 32 x 64 fp32 sums of the peers' partials
  uint32_t* rs_flag_local;             // [ws][rs_max_tiles]
  uint32_t* rs_flag_peer[MAX_WORLD];
  int32_t rs_max_tiles;
  int32_t rs_slot_rows;                // rows_per_rank rounded up to whole 128-row tiles
  int32_t rs_arena_tma;                // bf16 partials: blocked arena written by bulk copies
  int32_t rs_lag;                      // own row block j is scheduled this many row blocks after the peers' j (0: RS_LAG)
  float reduce_scale;                  // 1 for sum, 1/ws for avg
  // ---- common
  uint32_t epoch;
  uint32_t* status;
  long long timeout_cycles;
  // ---- optional timeline (apk_set_trace): TRACE_FIELDS u64 per (CTA, local tile), null when off
  unsigned long long* trace;
  int32_t trace_tiles;                 // records per CTA
};

// Fields of one timeline record. Times are %globaltimer nanoseconds, waits are SM cycles.
enum TraceField : int {
  TR_TILE = 0,          // producer: global tile index + 1 (0: record unused)
  TR_LOAD_T = 1,        // producer: first load of the tile issued
  TR_READY_WAIT = 2,    // producer: cycles waiting for gathered rows (all-gather mode)
  TR_EMPTY_WAIT = 3,    // producer: cycles waiting for free pipeline stages
  TR_MMA_T = 4,         // MMA thread: first MMA of the tile issued
  TR_FULL_WAIT = 5,     // MMA thread: cycles waiting for operands
  TR_TEMPTY_WAIT = 6,   // MMA thread: cycles waiting for a free accumulator
  TR_COMMIT_T = 7,      // MMA thread: the tile's last MMA issued and committed
  TR_TFULL_T = 8,       // epilogue: accumulator complete
  TR_PARTIAL_WAIT = 9,  // epilogue: cycles waiting for the peers' partials (reduce-scatter, own tile)
  TR_EPI_END_T = 10,    // epilogue: the tile's stores issued
  TR_PUBLISH = 11,      // epilogue: cycles inside flag publication during this tile
  TR_FLAGS_T = 12,      // summing warps: all peers' flags of an own tile acquired
  TR_SUMS_T = 13,       // summing warps: sums of an own tile written
  TR_CTA_BEGIN_T = 14,  // record 0 of a CTA: CTA start in ns; record 1: the same instant in SM cycles
  TR_CTA_END_T = 15,    // record 0: CTA end in ns; record 1: in SM cycles (cycles / ns = the SM clock in GHz)
  TRACE_FIELDS = 16
};

// Pipeline stages are handed back to the producer in groups of RELEASE_EVERY k-blocks (one
// tcgen05.commit per group instead of one per k-block). The single MMA-issuing thread is the
// scarce resource of this kernel: measured on B200, a tcgen05.mma (cta_group::2) costs it about 75
// cycles, a commit 140-170 and a barrier wait 55-85, against 128 tensor-pipe cycles per 256 x 256 x 16
// MMA; with four MMAs per commit and wait the thread, not the pipe, sets the pace (about 690 cycles
// per k-block against 512), with eight it stays ahead of the pipe.
template <int STAGES>
struct ReleaseEvery {
  static constexpr int value = (STAGES % 2 == 0 && STAGES >= 6) ? 2 : 1;
};

template <int BN, int STAGES, bool PAIR = false>
struct SmemLayout {
  static constexpr int A_BYTES = BM * ROW_BYTES;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * ROW_BYTES;   // a CTA of a pair holds half of B's columns
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STG_OFF = STAGES * STAGE_BYTES;              // epilogue staging, 1024-aligned
  static constexpr int STG_SLOT_BYTES = 32 * ROW_BYTES;             // 32 rows x 128 bytes: one warp's block
  static constexpr int STG_BUF_BYTES = EPI_WARPS * STG_SLOT_BYTES;  // two buffers of four slots [buffer][quarter]: the four
                                                                    // quarters of a buffer are contiguous (one 16 KiB bulk copy)
  static constexpr int BAR_OFF = STG_OFF + 2 * STG_BUF_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 5;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int TOTAL = MISC_OFF + 32 + 1024;  // + alignment slack
};

struct TileInfo {
  int chunk;        // which rank's rows (AG: source rank, RS: destination rank)
  int mt;           // row block inside the chunk
  int b;            // which B / output
  int n0;           // first column inside output b
  int tile_in_chunk;
  int rows_valid;   // rows of this tile that exist
  int n_valid;      // columns of this tile that exist
};

struct Sched {
  int nt_b[MAX_B];
  int nt_total;
  int mt_per_chunk;
  int tiles_per_chunk;   // 128-row tiles per chunk (indexing of flags and arena blocks)
  int units_per_chunk;   // scheduling units per chunk: tiles, or pairs of vertically adjacent tiles
  int num_chunks;
  int total_tiles;       // scheduling units in the whole problem
};

template <int BN, bool PAIR = false>
__host__ __device__ __forceinline__ Sched make_sched(const KParams& p) {
  Sched s;
  s.nt_total = 0;
#pragma unroll
  for (int b = 0; b < MAX_B; ++b) {
    s.nt_b[b] = (b < p.nB) ? (p.N[b] + BN - 1) / BN : 0;
    s.nt_total += s.nt_b[b];
  }
  s.mt_per_chunk = (p.rows_per_rank + BM - 1) / BM;
  s.tiles_per_chunk = s.mt_per_chunk * s.nt_total;
  s.units_per_chunk = (PAIR ? s.mt_per_chunk / 2 : s.mt_per_chunk) * s.nt_total;
  s.num_chunks = (p.mode == MODE_PLAIN || p.ag_ksplit) ? 1 : p.ws;
  s.total_tiles = s.units_per_chunk * s.num_chunks;
  return s;
}

// Tile order. Rows of the local rank's chunk form one block of tiles_per_chunk tiles (first in
// all-gather mode, last in reduce-scatter mode). The other ranks' chunks are interleaved row
// block by row block: (row block 0 of rank+1, row block 0 of rank+2, ..., row block 1 of rank+1, ...),
// so that at any moment a GPU exchanges data with all of its peers at once. On an NVSwitch
// fabric this keeps every GPU's ingress and egress busy even when the ranks drift apart,
// which a strict "one peer per step" order does not.
// With PAIR a unit is two vertically adjacent tiles (same columns); `crank` (0 or 1) picks this CTA's.
template <int BN, bool PAIR = false>
__host__ __device__ __forceinline__ TileInfo decode_tile(const KParams& p, const Sched& s, int t, int crank = 0) {
  TileInfo ti;
  int nt;
  if (p.mode == MODE_PLAIN || p.ws == 1 || p.ag_ksplit) {
    ti.chunk = (p.mode == MODE_PLAIN || p.ag_ksplit) ? 0 : p.rank;
    ti.mt = t / s.nt_total;
    nt = t - ti.mt * s.nt_total;
  } else if (p.mode == MODE_AG) {
    if (t < s.units_per_chunk) {
      ti.chunk = p.rank;
      ti.mt = t / s.nt_total;
      nt = t - ti.mt * s.nt_total;
    } else {
      const int r = t - s.units_per_chunk;
      const int per_mt = s.nt_total * (p.ws - 1);
      ti.mt = r / per_mt;
      const int rr = r - ti.mt * per_mt;
      const int step = rr / s.nt_total;                 // 0 .. ws-2
      nt = rr - step * s.nt_total;
      ti.chunk = (p.rank + 1 + step) % p.ws;
    }
  } else {
    // Reduce-scatter: row block j of the local rank's chunk follows RS_LAG row blocks behind the
    // peers' row block j (whose partials for it are then on their way or already here), so the
    // NVLink traffic is spread over the whole kernel instead of stopping when the own chunk starts.
    const int U = s.nt_total;                    // units per row block of one chunk
    const int R = U * (p.ws - 1);                // remote units per row block
    const int rows = s.units_per_chunk / U;      // row blocks (or pairs of them)
    const int want = p.rs_lag > 0 ? p.rs_lag : RS_LAG;
    const int lag = rows < want ? rows : want;
    const int head = lag * R;
    const int body = (rows - lag) * (R + U);
    int remote_r = -1, own_r = -1;               // index inside the remote / own sequence
    if (t < head) {
      remote_r = t;
    } else if (t < head + body) {
      const int t2 = t - head;
      const int g = t2 / (R + U);
      const int w = t2 - g * (R + U);
      if (w < R) remote_r = (lag + g) * R + w; else own_r = g * U + (w - R);
    } else {
      own_r = (rows - lag) * U + (t - head - body);
    }
    if (own_r >= 0) {
      ti.chunk = p.rank;
      ti.mt = own_r / U;
      nt = own_r - ti.mt * U;
    } else {
      ti.mt = remote_r / R;
      const int rr = remote_r - ti.mt * R;
      const int step = rr / U;                          // 0 .. ws-2
      nt = rr - step * U;
      ti.chunk = (p.rank + 1 + step) % p.ws;
    }
  }
  if (PAIR) ti.mt = 2 * ti.mt + crank;
  ti.tile_in_chunk = ti.mt * s.nt_total + nt;
  ti.b = 0;
#pragma unroll
  for (int b = 0; b < MAX_B - 1; ++b) {
    if (ti.b == b && nt >= s.nt_b[b]) {
      nt -= s.nt_b[b];
      ti.b = b + 1;
    }
  }
  ti.n0 = nt * BN;
  const int rows_left = p.rows_per_rank - ti.mt * BM, cols_left = p.N[ti.b] - ti.n0;
  ti.rows_valid = rows_left < BM ? rows_left : BM;
  ti.n_valid = cols_left < BN ? cols_left : BN;
  return ti;
}

// Number of 4 KiB pieces the all-gather pull splits row block `mt` of a chunk into.
__device__ __forceinline__ int ag_tile_pieces(const KParams& p, int mt) {
  const long long tile_bytes = (long long)BM * p.K * p.elem_bytes;
  const long long start = (long long)mt * tile_bytes;
  long long len = p.ag_chunk_bytes - start;
  if (len > tile_bytes) len = tile_bytes;
  return (int)((len + PIECE_BYTES - 1) / PIECE_BYTES);
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Timeline slot `field` of this CTA's local tile `lt`; null when tracing is off or the buffer is full.
__device__ __forceinline__ unsigned long long* trace_slot(const KParams& p, uint32_t lt, int field) {
  if (p.trace == nullptr || lt >= (uint32_t)p.trace_tiles) return nullptr;
  return p.trace + ((size_t)blockIdx.x * p.trace_tiles + lt) * TRACE_FIELDS + field;
}
__device__ __forceinline__ void trace_put(const KParams& p, uint32_t lt, int field, unsigned long long v) {
  unsigned long long* s = trace_slot(p, lt, field);
  if (s != nullptr) *s = v;
}

__device__ __forceinline__ void set_status(const KParams& p, uint32_t code, uint32_t detail) {
  atomicCAS(p.status, 0u, code | (detail << 8));
}

// Bounded mbarrier wait. Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const KParams& p, volatile uint32_t* abort_flag) {
  uint32_t spins = 0;
  long long t0 = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > p.timeout_cycles) {
        set_status(p, ST_TIMEOUT_MBAR, bar & 0xffffu);
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// Bounded wait until the u32 at `flag` has reached `target` (wrap-safe). `sys` selects the scope.
template <bool SYS>
__device__ __forceinline__ bool flag_wait(const uint32_t* flag, uint32_t target, const KParams& p,
                                          volatile uint32_t* abort_flag, uint32_t code, uint32_t detail) {
  uint32_t spins = 0;
  long long t0 = 0;
  while (true) {
    const uint32_t v = SYS ? ptx::ld_acquire_sys(flag) : ptx::ld_acquire_gpu(flag);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++spins & 0x3fu) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > p.timeout_cycles) {
        set_status(p, code, detail);
        *abort_flag = 1;
        return false;
      }
      __nanosleep(64);
    }
  }
}

// Bounded wait until a shared-memory counter written by other warps of the CTA reaches `target`.
__device__ __forceinline__ bool smem_count_wait(volatile uint32_t* ctr, uint32_t target, const KParams& p,
                                                volatile uint32_t* abort_flag) {
  uint32_t spins = 0;
  long long t0 = 0;
  while ((int32_t)(*ctr - target) < 0) {
    if ((++spins & 0x3fu) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2 * p.timeout_cycles) {   // the waiting warp it depends on reports first
        set_status(p, ST_TIMEOUT_PARTIAL, 0xffu);
        *abort_flag = 1;
        return false;
      }
      __nanosleep(32);
    }
  }
  __threadfence_block();
  return true;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Two fp32 values rounded to one 32-bit pair of bf16 (f16 == false) or IEEE half.
__device__ __forceinline__ uint32_t pack16(float lo, float hi, bool f16) {
  if (f16) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  return pack_bf16(lo, hi);
}

// Writes `nvalid` (multiple of 8 for bf16, 4 for fp32; <= 32) consecutive outputs of one row.
__device__ __forceinline__ void store_row32(void* dst, const float (&v)[32], int nvalid, bool fp32, bool f16 = false) {
  if (fp32) {
    float4* d = reinterpret_cast<float4*>(dst);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j * 4 < nvalid) d[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  } else {
    uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j * 8 < nvalid) {
        uint4 q;
        q.x = pack16(v[8 * j + 0], v[8 * j + 1], f16);
        q.y = pack16(v[8 * j + 2], v[8 * j + 3], f16);
        q.z = pack16(v[8 * j + 4], v[8 * j + 5], f16);
        q.w = pack16(v[8 * j + 6], v[8 * j + 7], f16);
        d[j] = q;
      }
    }
  }
}

// v += the 32 values of one row of a partial that a peer left in the local arena.
__device__ __forceinline__ void add_row32(const void* src, float (&v)[32], int nvalid, bool fp32) {
  if (fp32) {
    const float4* s = reinterpret_cast<const float4*>(src);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j * 4 < nvalid) {
        const float4 q = __ldcg(s + j);
        v[4 * j] += q.x; v[4 * j + 1] += q.y; v[4 * j + 2] += q.z; v[4 * j + 3] += q.w;
      }
    }
  } else {
    const uint4* s = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j * 8 < nvalid) {
        const uint4 q = __ldcg(s + j);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[8 * j + 2 * e] += __uint_as_float(w[e] << 16);
          v[8 * j + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
        }
      }
    }
  }
}

// One warp copies up to 4 KiB (n16 16-byte words) of local memory src -> dst (and dst2 when given).
__device__ __forceinline__ void copy_piece(const uint8_t* src, uint8_t* dst, uint8_t* dst2, int n16, int lane) {
  uint4 r[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = u * 32 + lane;
    if (i < n16) {
      r[u] = __ldcg(reinterpret_cast<const uint4*>(src) + i);
    }
  }
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = u * 32 + lane;
    if (i < n16) {
      reinterpret_cast<uint4*>(dst)[i] = r[u];
      if (dst2 != nullptr) reinterpret_cast<uint4*>(dst2)[i] = r[u];
    }
  }
}

// PAIR: the grid is made of clusters of two CTAs; a pair works on two vertically adjacent tiles
// (256 rows x BN columns) with one tcgen05.mma.cta_group::2 stream issued by the CTA of cluster
// rank 0. Each CTA loads its own 128 rows of A and HALF of B's columns (32 KiB instead of 48 KiB
// per k-block from L2, the bound of the single-CTA kernel), keeps its 128 x BN accumulator in its
// own TMEM and runs its own epilogue and communication warps exactly as without PAIR.
// TRACE: the timeline instrumentation is compiled in. It is a template parameter and not a run-time test
// because the MMA-issuing thread sets the pace of the kernel: a few extra instructions in its loop, even
// never-taken branches, cost several percent of the whole GEMM (measured). Launches made while a timeline
// buffer is set use the TRACE instances; all others carry none of it.
template <int BN, int STAGES, bool FP8, bool PAIR, bool TRACE = false>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_fused_kernel(const __grid_constant__ KParams p) {
  using L = SmemLayout<BN, STAGES, PAIR>;
  constexpr int BKE = FP8 ? 128 : 64;           // K elements per stage (128 bytes)
  constexpr int UMMA_K = FP8 ? 32 : 16;         // K elements per tcgen05.mma (32 bytes)
  constexpr int KSTEPS = BKE / UMMA_K;          // 4
  constexpr int NPB = FP8 ? 128 : 64;           // N elements per TMA box when B is N-major
  constexpr int RE = ReleaseEvery<STAGES>::value;   // k-blocks per stage release
  constexpr uint32_t TMEM_COLS = 2 * BN <= 32 ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::MISC_OFF);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF + 4);
  volatile uint32_t* epi_verdict = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF + 8);  // [2]
  // reduce-scatter: how many of this CTA's own tiles have had their peers' partials summed
  volatile uint32_t* sums_done = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF + 16);
  // reduce-scatter: the summing warps' shared decision to go on (written by one thread per tile)
  volatile uint32_t* sum_verdict = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF + 20);   // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const Sched sched = make_sched<BN, PAIR>(p);
  const int crank = PAIR ? (int)ptx::cluster_ctarank() : 0;          // rank inside the pair
  const int tile_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int kb_per_shard = (p.K + BKE - 1) / BKE;
  const int num_kb = p.ag_ksplit ? kb_per_shard * p.ws : kb_per_shard;   // K-split: every rank's K-slice in turn

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), PAIR ? 2 : 1);   // pair: both CTAs' producers arrive on rank 0's barrier
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), PAIR ? 2 * EPI_WARPS : EPI_WARPS);   // pair: both CTAs' epilogues
    }
    ptx::mbar_init(drain_bar, 1);
    *abort_flag = 0;
    *sums_done = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(tmem_ptr_smem), TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(tmem_ptr_smem), TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  if (PAIR) ptx::cluster_sync(); else __syncthreads();   // pair: the other CTA's barriers are initialised too
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ============================================================ TMA producer
    if (lane == 0) {
      ptx::tma_prefetch_desc(&p.tmA0);
      if (p.mode == MODE_AG) ptx::tma_prefetch_desc(&p.tmA1);
      for (int b = 0; b < p.nB; ++b) ptx::tma_prefetch_desc(&p.tmB[b]);
      uint32_t it = 0;       // k-block counter over the CTA's lifetime
      uint32_t pstage = 0, pphase = 0;   // = it % STAGES and (it / STAGES) & 1, kept as counters
      uint32_t lt = 0;       // local tile counter
      constexpr bool tracing = TRACE;
      bool ok = true;
      if (tracing) {
        trace_put(p, 0, TR_CTA_BEGIN_T, globaltimer_ns());
        trace_put(p, 1, TR_CTA_BEGIN_T, (unsigned long long)clock64());
      }
      for (int t = tile_first; t < sched.total_tiles && ok; t += tile_step, ++lt) {
        const TileInfo ti = decode_tile<BN, PAIR>(p, sched, t, crank);
        long long tr_ready = 0, tr_empty = 0;
        const CUtensorMap* tmA = &p.tmA0;
        int arow = ti.mt * BM;
        int bcol = ti.n0;     // first column of B for this tile
        if (p.ag_ksplit) {
          // handled per k-block below: the source rank changes along K
        } else if (p.mode == MODE_AG && ti.chunk != p.rank) {
          tmA = &p.tmA1;
          arow += ti.chunk * p.rows_per_rank;
          const uint32_t expect = (uint32_t)ag_tile_pieces(p, ti.mt) + (p.ag_has_scale ? 1u : 0u);
          const long long c0 = tracing ? clock64() : 0;
          ok = flag_wait<false>(p.ready + ti.chunk * sched.mt_per_chunk + ti.mt, expect, p, abort_flag,
                                ST_TIMEOUT_READY, (uint32_t)ti.chunk);
          if (tracing) tr_ready += clock64() - c0;
          if (!ok) break;
          ptx::fence_proxy_async_global();
        } else if (p.mode == MODE_RS) {
          if (p.rs_colsplit) bcol += ti.chunk * p.N[0]; else arow += ti.chunk * p.rows_per_rank;
        }
        const bool nmajor = p.b_nmajor[ti.b] != 0;
        const CUtensorMap* tmB = &p.tmB[ti.b];
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)pstage;
          const uint32_t ph = pphase;
          if (++pstage == (uint32_t)STAGES) { pstage = 0; pphase ^= 1u; }
          int ka = kb * BKE, kbB = kb * BKE;     // K coordinates in A and in B
          if (p.ag_ksplit) {
            // K-slice of rank (rank + step): own slice first, then the peers' as they arrive
            const int step = kb / kb_per_shard;
            const int src = (p.rank + step) % p.ws;
            ka = (kb - step * kb_per_shard) * BKE;
            kbB = src * p.K + ka;
            if (ka == 0) {
              tmA = (src == p.rank) ? &p.tmA0 : &p.tmA1;
              arow = ti.mt * BM + ((src == p.rank) ? 0 : src * p.rows_per_rank);
              if (src != p.rank) {
                const uint32_t expect = (uint32_t)ag_tile_pieces(p, ti.mt);
                const long long c0 = tracing ? clock64() : 0;
                ok = flag_wait<false>(p.ready + src * sched.mt_per_chunk + ti.mt, expect, p, abort_flag,
                                      ST_TIMEOUT_READY, (uint32_t)src);
                if (tracing) tr_ready += clock64() - c0;
                if (!ok) break;
                ptx::fence_proxy_async_global();
              }
            }
          }
          {
            // stages come back in groups of RE: only the first stage of a group waits
            const long long c0 = tracing ? clock64() : 0;
            if (s % RE == 0) ok = mbar_wait(empty_bar(s / RE), ph ^ 1u, p, abort_flag);
            if (tracing) {
              tr_empty += clock64() - c0;
              if (kb == 0) {
                trace_put(p, lt, TR_TILE, (unsigned long long)t + 1ull);
                trace_put(p, lt, TR_LOAD_T, globaltimer_ns());
              }
            }
          }
          if (!ok) break;
          const uint32_t a_dst = smem_base + s * L::STAGE_BYTES;
          const uint32_t b_dst = a_dst + L::A_BYTES;
          if (PAIR) {
            // this CTA's A rows and its half of B's columns; bytes are counted on rank 0's barrier
            const uint32_t fb = ptx::mapa(full_bar(s), 0);
            const int nb = bcol + crank * (BN / 2);
            ptx::mbar_expect_tx_cluster(fb, L::STAGE_BYTES);
            ptx::tma_load_2d_pair(a_dst, tmA, fb, ka, arow);
            if (!nmajor) {
              ptx::tma_load_2d_pair(b_dst, &p.tmBp[ti.b], fb, kbB, nb);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 2 / NPB; ++j) {
                ptx::tma_load_2d_pair(b_dst + j * (BKE * ROW_BYTES), tmB, fb, nb + j * NPB, kbB);
              }
            }
          } else {
            ptx::mbar_expect_tx(full_bar(s), L::STAGE_BYTES);
            ptx::tma_load_2d(a_dst, tmA, full_bar(s), ka, arow);
            if (!nmajor) {
              ptx::tma_load_2d(b_dst, tmB, full_bar(s), kbB, bcol);
            } else {
#pragma unroll
              for (int j = 0; j < BN / NPB; ++j) {
                ptx::tma_load_2d(b_dst + j * (BKE * ROW_BYTES), tmB, full_bar(s), bcol + j * NPB, kbB);
              }
            }
          }
        }
        if (tracing) {
          trace_put(p, lt, TR_READY_WAIT, (unsigned long long)tr_ready);
          trace_put(p, lt, TR_EMPTY_WAIT, (unsigned long long)tr_empty);
        }
      }
      // Drain: every load this thread armed has either landed or is given a bounded time to.
      const uint32_t last = (PAIR && crank != 0) ? 0u : it;   // (rank 1 of a pair has no full barriers of its own)
      const uint32_t first = last > (uint32_t)STAGES ? last - STAGES : 0u;
      for (uint32_t i = first; i < last; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1u;
        uint32_t spins = 0;
        while (!ptx::mbar_try_wait(full_bar(s), ph) && ++spins < (1u << 16)) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ============================================================ MMA issuer
    // The whole warp walks the loop (waits, stage bookkeeping and descriptor arithmetic are the same in all
    // lanes, so they can stay in the uniform datapath) and ONE elected lane issues the tcgen05 instructions:
    // with the loop inside a single-lane branch every operand of every MMA had to be moved over from that
    // lane's registers first.
    if (crank == 0) {
      // Shared-memory matrix descriptor: version 1 (bit 46), 128-byte swizzle (2 << 61),
      // stride byte offset 1024 (8 rows x 128 B) in 16-byte units at bit 32.
      const uint64_t desc_common = (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(1024 >> 4) << 32);
      const uint64_t desc_kmajor = desc_common | (uint64_t(1) << 16);
      const uint64_t desc_nmajor = desc_common | (uint64_t((BKE * ROW_BYTES) >> 4) << 16);
      // Instruction descriptor: fp32 accumulate, A/B format (bf16 = 1, e4m3 = 0), M = 128.
      const uint32_t fmt = (FP8 || p.in_f16) ? 0u : 1u;   // kind::f16: 0 = half, 1 = bf16; kind::f8f6f4: 0 = e4m3
      const uint32_t idesc_base = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t((PAIR ? 2 * BM : BM) >> 4) << 24);
      uint32_t lt = 0;  // local tile counter
      constexpr bool tracing = TRACE;
      bool ok = true;
      // The loop below is kept short on purpose (see ReleaseEvery): stage and phase are running counters,
      // the barrier addresses of both CTAs are computed once, and the next stage's `full` barrier is
      // probed (non-blocking) before this stage's MMAs are issued, so that its latency is hidden.
      uint32_t stage = 0, phase = 0;
      const uint32_t full0 = full_bar(0);
      const uint32_t empty_c0 = PAIR ? ptx::mapa(empty_bar(0), 0) : empty_bar(0);
      const uint32_t empty_c1 = PAIR ? ptx::mapa(empty_bar(0), 1) : 0u;
      const uint32_t tfull_c0 = PAIR ? ptx::mapa(tfull_bar(0), 0) : tfull_bar(0);
      const uint32_t tfull_c1 = PAIR ? ptx::mapa(tfull_bar(0), 1) : 0u;
      const uint32_t a_lo0 = (smem_base >> 4) & 0x3fffu;
      const uint32_t b_lo0 = ((smem_base + L::A_BYTES) >> 4) & 0x3fffu;
      // every decision that steers the loop is made warp-uniform (votes), so that all lanes reach every elect
      bool ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0, 0u));
      for (int t = tile_first; t < sched.total_tiles && ok; t += tile_step, ++lt) {
        const TileInfo ti = decode_tile<BN, PAIR>(p, sched, t, crank);
        const uint32_t acc = lt & 1u;
        const uint32_t aph = (lt >> 1) & 1u;
        long long tr_full = 0;
        {
          const long long c0 = tracing ? clock64() : 0;
          ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(acc), aph ^ 1u, p, abort_flag));
          if (tracing && lane == 0) trace_put(p, lt, TR_TEMPTY_WAIT, (unsigned long long)(clock64() - c0));
        }
        if (!ok) break;
        ptx::tc_fence_after();
        const bool nmajor = p.b_nmajor[ti.b] != 0;
        const int n_eff = PAIR ? BN : min(BN, (ti.n_valid + 15) & ~15);   // a pair splits N evenly, so it is fixed
        const uint32_t idesc = idesc_base | (nmajor ? (1u << 16) : 0u) | (uint32_t(n_eff >> 3) << 17);
        const uint32_t d_tmem = tmem_base + acc * BN;
        const uint64_t bdesc_hi = nmajor ? desc_nmajor : desc_kmajor;
        const uint32_t bstep = nmajor ? uint32_t((UMMA_K * ROW_BYTES) >> 4) : 2u;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ready) {
            const long long c0 = tracing ? clock64() : 0;
            ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8u * stage, phase, p, abort_flag));
            if (tracing) tr_full += clock64() - c0;
            if (!ok) break;
          }
          if (tracing && kb == 0 && lane == 0) trace_put(p, lt, TR_MMA_T, globaltimer_ns());
          ptx::tc_fence_after();
          const uint32_t s = stage;
          if (++stage == (uint32_t)STAGES) { stage = 0; phase ^= 1u; }
          ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0 + 8u * stage, phase));   // the NEXT k-block's operands (may belong to the next tile)
          const uint64_t adesc = desc_kmajor | uint64_t(a_lo0 + s * (uint32_t)(L::STAGE_BYTES >> 4));
          const uint64_t bdesc = bdesc_hi | uint64_t(b_lo0 + s * (uint32_t)(L::STAGE_BYTES >> 4));
          if (ptx::elect_one()) {
#pragma unroll
          for (int k = 0; k < KSTEPS; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            if (PAIR) {
              if (FP8) ptx::mma_f8_pair(d_tmem, adesc + 2u * k, bdesc + bstep * k, idesc, accum);
              else ptx::mma_f16_pair(d_tmem, adesc + 2u * k, bdesc + bstep * k, idesc, accum);
            } else if (FP8) {
              ptx::mma_f8(d_tmem, adesc + 2u * k, bdesc + bstep * k, idesc, accum);
            } else {
              ptx::mma_f16(d_tmem, adesc + 2u * k, bdesc + bstep * k, idesc, accum);
            }
          }
          if (s % RE == RE - 1) {   // the group of stages is free again (in both CTAs of a pair)
            if (PAIR) {
              ptx::tc_commit_pair(empty_c0 + 8u * (s / RE));
              ptx::tc_commit_pair(empty_c1 + 8u * (s / RE));
            } else {
              ptx::tc_commit(empty_c0 + 8u * (s / RE));
            }
          }
          }   // elected lane
        }
        if (ok && ptx::elect_one()) {
          if (PAIR) {
            ptx::tc_commit_pair(tfull_c0 + 8u * acc);
            ptx::tc_commit_pair(tfull_c1 + 8u * acc);
          } else {
            ptx::tc_commit(tfull_c0 + 8u * acc);
          }
        }
        if (tracing && lane == 0) {
          trace_put(p, lt, TR_FULL_WAIT, (unsigned long long)tr_full);
          trace_put(p, lt, TR_COMMIT_T, globaltimer_ns());
        }
      }
      // Make sure nothing the elected lane issued is still running before TMEM is freed.
      __syncwarp();
      if (ptx::elect_one()) {
        if (PAIR) ptx::tc_commit_pair(ptx::mapa(drain_bar, 0)); else ptx::tc_commit(drain_bar);
      }
      uint32_t spins = 0;
      while (!ptx::mbar_try_wait(drain_bar, 0) && ++spins < (1u << 20)) {
      }
    }
    __syncwarp();
  } else if (warp < 2 + EPI_WARPS) {
    // ============================================================ epilogue
    const int quarter = warp & 3;                   // TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const bool epi_leader = (warp == 2 && lane == 0);
    const uint32_t stg_all = smem_base + L::STG_OFF;
    // this warp's slot in staging buffer b
    auto slot = [&](uint32_t b) { return stg_all + b * (uint32_t)L::STG_BUF_BYTES + (uint32_t)quarter * (uint32_t)L::STG_SLOT_BYTES; };
    // fp32 sums of an own reduce-scatter block: 32 rows x 256 bytes spread over this warp's two slots
    // (16-byte unit u of row r: slot u >> 3, byte r * 128 + (u & 7) * 16)
    auto sum_addr = [&](uint32_t row, uint32_t unit) { return slot(unit >> 3) + row * (uint32_t)ROW_BYTES + ((unit & 7u) << 4); };
    uint32_t stg_count = 0;
    bool prev_coop = false;   // the previous tile left as cooperative 16 KiB copies issued by the leader
    uint32_t lt = 0;
    constexpr bool tracing = TRACE;
    // Reduce-scatter: tiles sent to their owners and not yet announced, oldest first (the same
    // values in all 4 warps). Up to four tiles stay in flight and flags are released two tiles at
    // a time behind ONE system-scope fence: a fence costs a round trip over a busy NVLink, so it
    // must neither be paid per tile nor wait for the newest stores.
    uint32_t* pq_flag[4] = {nullptr, nullptr, nullptr, nullptr};
    int pq_newer[4] = {0, 0, 0, 0};   // bulk groups this warp committed after the tile's own
    bool pq_gen[4] = {false, false, false, false};
    int pq_n = 0;
    auto publish_oldest = [&](int count) {   // count = 1 or 2, count <= pq_n
      // Every store of these tiles complete, then the flags.
      // Bulk copies are all issued, and their groups tracked, by the leader (warp 2, lane 0). It only waits
      // for their completion; the system-scope fence and the flag stores are the herald's (warp 3, lane 0),
      // which the leader meets at a two-warp barrier: a fence.sys waits for whatever its own thread has in
      // flight, and the leader always has the newest tile's copies on the wire (measured at 8 ranks: 8 us per
      // fence in the leader). Direct stores (fp32 partials) are each thread's own, fenced by itself, then the
      // four warps meet and the leader publishes.
      const int newer = pq_newer[count - 1];
      bool generic = pq_gen[0] || (count == 2 && pq_gen[1]);
      const bool herald = (warp == 3 && lane == 0);
      const long long c0 = (tracing && (epi_leader || herald)) ? clock64() : 0;
      if (generic) {
        __threadfence_system();
        ptx::named_bar_sync(2, EPI_WARPS * 32);
      } else if (warp == 2 || warp == 3) {
        if (epi_leader) ptx::bulk_wait_group_upto(newer);
        ptx::named_bar_sync(4, 64);
      }
      if (generic ? epi_leader : herald) {
        __threadfence_system();
        ptx::st_relaxed_sys(pq_flag[0], p.epoch);
        if (count == 2) ptx::st_relaxed_sys(pq_flag[1], p.epoch);
      }
      if (tracing && (epi_leader || herald)) {
        unsigned long long* tslot = trace_slot(p, lt, TR_PUBLISH);
        if (tslot != nullptr) atomicAdd(tslot, (unsigned long long)(clock64() - c0));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = i + count;
        pq_flag[i] = (j < 4) ? pq_flag[j < 4 ? j : 3] : nullptr;
        pq_newer[i] = (j < 4) ? pq_newer[j < 4 ? j : 3] : 0;
        pq_gen[i] = (j < 4) ? pq_gen[j < 4 ? j : 3] : false;
      }
      pq_n -= count;
    };
    auto publish_pending = [&]() {
      while (pq_n > 0) publish_oldest(pq_n >= 2 ? 2 : 1);
    };
    auto note_commit = [&]() {
#pragma unroll
      for (int i = 0; i < 4; ++i) ++pq_newer[i];   // entries beyond pq_n are reset when they are filled
    };
    auto push_pending = [&](uint32_t* flag, bool generic) {
      if (pq_n == 4) publish_oldest(2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i == pq_n) { pq_flag[i] = flag; pq_newer[i] = 0; pq_gen[i] = generic; }
      }
      ++pq_n;
    };
    uint32_t own_seen = 0;   // own reduce-scatter tiles this CTA has finished
    for (int t = tile_first; t < sched.total_tiles; t += tile_step, ++lt) {
      const TileInfo ti = decode_tile<BN, PAIR>(p, sched, t, crank);
      const uint32_t acc = lt & 1u;
      const uint32_t aph = (lt >> 1) & 1u;
      const bool row_ok = row_in_tile < ti.rows_valid;
      const int chunk_row = ti.mt * BM + row_in_tile;                   // row inside the chunk
      const long long grow = (p.rs_colsplit ? 0LL : (long long)ti.chunk * p.rows_per_rank) + chunk_row;  // row of the full matrix
      const int b = ti.b;
      const bool own = (p.mode != MODE_RS) || (ti.chunk == p.rank);

      // Before waiting on the peers, announce what this CTA still owes them: two ranks that each
      // held back their last partial while waiting for the other's would wait forever.
      if (p.mode == MODE_RS && own) publish_pending();
      // Bulk-copy tiles: all but the newest are announced here, by the leader alone, before it waits for the
      // next accumulator. Their copies were issued at least a tile's time ago (measured at 8 ranks: a 16 KiB
      // copy takes about 10 us to be acknowledged when every GPU is sending), so the leader hardly waits,
      // and the owner learns of a partial one tile after it was sent instead of several.
      if (p.mode == MODE_RS && p.rs_arena_tma != 0) {
        while (pq_n > 1) publish_oldest(pq_n > 2 ? 2 : 1);
      }
      // One thread does the waiting (peers' partials for a tile this rank owns, then the
      // accumulator); its verdict is shared so that all four warps leave the loop together.
      const bool coop = (p.mode == MODE_RS) && !own && p.rs_arena_tma != 0;   // this tile leaves as cooperative 16 KiB copies
      if (coop && !prev_coop) {
        // this warp's own tiled stores must have finished reading its staging slots
        if (lane == 0) ptx::bulk_wait_group_read<0>();
        __syncwarp();
      }
      if (epi_leader) {
        bool good = true;
        // the other warps are about to reuse slots that the leader's cooperative copies may still be reading
        if (prev_coop && !coop) ptx::bulk_wait_group_read<0>();
        const long long c0 = tracing ? clock64() : 0;
        if (p.mode == MODE_RS && own && p.ws > 2 && p.rs_arena_tma != 0) {
          // the communication warps acquire the peers' flags and leave the sum of their partials
          good = smem_count_wait(sums_done, own_seen + 1u, p, abort_flag);
        } else if (p.mode == MODE_RS && own && p.ws > 1) {
          for (int src = 0; src < p.ws && good; ++src) {
            if (src == p.rank) continue;
            good = flag_wait<true>(p.rs_flag_local + (size_t)src * p.rs_max_tiles + ti.tile_in_chunk, p.epoch, p,
                                   abort_flag, ST_TIMEOUT_PARTIAL, (uint32_t)src);
          }
        }
        if (tracing) trace_put(p, lt, TR_PARTIAL_WAIT, (unsigned long long)(clock64() - c0));
        if (good) good = mbar_wait(tfull_bar(acc), aph, p, abort_flag);
        if (tracing) trace_put(p, lt, TR_TFULL_T, globaltimer_ns());
        epi_verdict[lt & 1u] = good ? 1u : 0u;
      }
      ptx::named_bar_sync(1, EPI_WARPS * 32);
      if (epi_verdict[lt & 1u] == 0u) break;
      ptx::tc_fence_after();

      // Row / tile constants of the scaled epilogue. Read only now: the gathered row scales of a
      // peer's chunk are in place once the accumulator that consumed those rows is complete.
      float sa = 1.0f;
      if (p.a_scale_mode == 1) {
        sa = __ldg(p.a_scale_full);
      } else if (p.a_scale_mode == 2 && row_ok) {
        if (p.mode == MODE_AG && p.a_scale_own != nullptr) {
          sa = (ti.chunk == p.rank) ? __ldg(p.a_scale_own + chunk_row) : __ldcg(p.ag_scale_gathered + grow);
        } else {
          sa = __ldg(p.a_scale_full + grow);
        }
      }
      const float* bs = p.b_scale[b];
      const int bs_mode = p.b_scale_mode[b];
      if (bs_mode == 1) sa *= __ldg(bs);
      const float rscale = (p.result_scale[b] != nullptr) ? __ldg(p.result_scale[b]) : 1.0f;
      const void* bias = p.bias[b];
      const bool scaled = (p.a_scale_mode != 0) || (bs_mode != 0) || (bias != nullptr) || (p.result_scale[b] != nullptr);


      const bool o32 = p.out_fp32[b] != 0;
      const bool o16h = p.out_f16[b] != 0;
      const int oes = o32 ? 4 : 2;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      const bool rs_remote = (p.mode == MODE_RS) && !own;
      // Stores go through shared memory and the TMA engine whenever that is possible: bf16, and
      // either all 128 rows exist (local outputs, tiled store clipped at N) or the target is a
      // peer's arena, which is laid out in whole 32 x 64 blocks so that every store over NVLink is
      // one linear 4 KiB bulk copy (row-strided 128-byte writes reach a fraction of the link rate).
      const bool use_tma = rs_remote ? (p.rs_arena_tma != 0) : (p.out_tma[b] != 0 && ti.rows_valid == BM);
      const CUtensorMap* tm_st = &p.tmOut[b];
      int st_row;  // first row this warp stores, in the coordinates of tm_st
      if (rs_remote) {
        st_row = 0;  // computed per 64-column group below
      } else if (p.mode == MODE_RS) {
        st_row = ti.mt * BM + quarter * 32;
      } else {
        st_row = ti.chunk * p.rows_per_rank + ti.mt * BM + quarter * 32;
      }
#pragma unroll 1
      for (int g = 0; g < BN / 64; ++g) {
        if (g * 64 >= ti.n_valid) break;   // uniform across the warp
        const uint32_t stg = slot(stg_count & 1u);
        // A tile this rank owns: the peers' bf16 partials of this 32-row x 64-column block are
        // summed first, with coalesced loads (lane i takes 16-byte chunks i, i+32, ... of each
        // 4 KiB block; row-per-thread loads reached a small fraction of the memory rate). The
        // fp32 sums go through both staging buffers (8 KiB) so that each thread can pick up its row.
        const bool own_any = (p.mode == MODE_RS) && own && p.ws > 1 && p.rs_arena_tma != 0;
        // With a single peer there is nothing to sum: its bf16 partial block is added as it arrived (a pre-summed
        // fp32 copy would cost three times the partial's bytes in extra memory traffic for a format conversion).
        const bool own_direct = own_any && p.ws == 2;
        const bool own_blocked = own_any && p.ws > 2;
        if ((use_tma && !coop) || own_any) {
          // the stores that last used the staging memory must have finished reading it
          if (lane == 0) {
            if (own_any) ptx::bulk_wait_group_read<0>(); else ptx::bulk_wait_group_read<1>();
          }
          __syncwarp();
        }
        if (own_direct) {
          // the peer's 4 KiB block of this warp's 32 rows x 64 columns, copied as it is (rows of 128 bytes, 16-byte
          // chunks XOR-swizzled by row, exactly as the sender staged it) into this warp's first staging slot
          const size_t peer_stride = (size_t)sched.tiles_per_chunk * (BN / 64) * 4 * (32 * ROW_BYTES);
          const uint8_t* pp = p.rs_arena_local + (size_t)(1 - p.rank) * peer_stride +
                              ((((size_t)ti.tile_in_chunk * (BN / 64) + g) * 4 + quarter) * (size_t)(32 * ROW_BYTES));
          uint4 u4[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) u4[i] = ptx::ld_cg_v4(pp + (size_t)(i * 32 + lane) * 16);
#pragma unroll
          for (int i = 0; i < 8; ++i) ptx::st_shared_v4(slot(0) + (uint32_t)(i * 32 + lane) * 16u, u4[i].x, u4[i].y, u4[i].z, u4[i].w);
          __syncwarp();
        }
        if (own_blocked) {
          // 8 KiB of fp32 sums for this warp's 32 rows x 64 columns, in the order of the bf16 blocks
          // they were summed from: 16-byte unit U holds half h = U & 1 of chunk L = U >> 1, which is
          // (row L / 8, stored position L % 8) = logical chunk (L % 8) ^ (row & 7). Coalesced loads,
          // then a 256-byte fp32 row per thread in shared memory, XOR-swizzled against bank conflicts.
          const uint8_t* sp = reinterpret_cast<const uint8_t*>(p.rs_sum_local) +
                              ((((size_t)ti.tile_in_chunk * (BN / 64) + g) * 4 + quarter) * (size_t)(64 * ROW_BYTES));
          uint4 u4[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) u4[i] = ptx::ld_cg_v4(sp + (size_t)(i * 32 + lane) * 16);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint32_t U = (uint32_t)(i * 32 + lane);
            const uint32_t Lc = U >> 1, h = U & 1u;
            const uint32_t row = Lc >> 3, sw = row & 7u;
            const uint32_t c = (Lc & 7u) ^ sw;
            ptx::st_shared_v4(sum_addr(row, (2u * c + h) ^ sw), u4[i].x, u4[i].y, u4[i].z, u4[i].w);
          }
          __syncwarp();
        }
        uint32_t packed[2][16];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int c = g * 2 + hf;
          if (c * 32 >= ti.n_valid) break;
          uint32_t raw[32];
          ptx::tmem_ld_32x32(t_row + c * 32, raw);
          ptx::tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          const int col0 = ti.n0 + c * 32;
          const int nvalid = min(32, p.N[b] - col0);
          if (scaled) {
            // per-column operands are the same for every row (broadcast loads); 8 columns at a time
            const bool full = (nvalid == 32);
            const bool bs_vec = (bs_mode == 2) && full && ((reinterpret_cast<uintptr_t>(bs + col0) & 15u) == 0);
            const bool bias_bf16 = (bias != nullptr) && !p.bias_fp32[b];
            const __nv_bfloat16* bias_h = reinterpret_cast<const __nv_bfloat16*>(bias) + col0;
            const float* bias_f = reinterpret_cast<const float*>(bias) + col0;
            const bool bias_vec = bias_bf16 && full && ((reinterpret_cast<uintptr_t>(bias_h) & 15u) == 0);
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              float cs[8], cb[8];
              if (bs_vec) {
                const float4 q0 = __ldg(reinterpret_cast<const float4*>(bs + col0) + 2 * j8);
                const float4 q1 = __ldg(reinterpret_cast<const float4*>(bs + col0) + 2 * j8 + 1);
                cs[0] = q0.x; cs[1] = q0.y; cs[2] = q0.z; cs[3] = q0.w; cs[4] = q1.x; cs[5] = q1.y; cs[6] = q1.z; cs[7] = q1.w;
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) cs[e] = (bs_mode == 2 && 8 * j8 + e < nvalid) ? __ldg(bs + col0 + 8 * j8 + e) : 1.0f;
              }
              if (bias_vec) {
                const uint4 q = __ldg(reinterpret_cast<const uint4*>(bias_h) + j8);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  cb[2 * e] = __uint_as_float(w[e] << 16);
                  cb[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                }
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const int j = 8 * j8 + e;
                  cb[e] = (bias == nullptr || j >= nvalid) ? 0.0f : (bias_bf16 ? __bfloat162float(__ldg(bias_h + j)) : __ldg(bias_f + j));
                }
              }
#pragma unroll
              for (int e = 0; e < 8; ++e) v[8 * j8 + e] = (v[8 * j8 + e] * sa * cs[e] + cb[e]) * rscale;
            }
          }
          if (p.mode == MODE_RS && own) {
            if (own_direct) {
              // this thread's row of the peer's partial, half `hf`: chunk c sits at position c ^ (row & 7)
              const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t c = (uint32_t)(hf * 4 + j);
                const float4 q = ptx::ld_shared_f4(slot(0) + (uint32_t)lane * (uint32_t)ROW_BYTES + ((c ^ sw) << 4));
                const uint32_t w[4] = {__float_as_uint(q.x), __float_as_uint(q.y), __float_as_uint(q.z), __float_as_uint(q.w)};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  v[8 * j + 2 * e] += __uint_as_float(w[e] << 16);
                  v[8 * j + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
                }
              }
            } else if (own_blocked) {
              // this thread's row of the fp32 sums, half `hf`
              const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t c = (uint32_t)(hf * 4 + j);
                const float4 s0 = ptx::ld_shared_f4(sum_addr((uint32_t)lane, (2u * c) ^ sw));
                const float4 s1 = ptx::ld_shared_f4(sum_addr((uint32_t)lane, (2u * c + 1u) ^ sw));
                v[8 * j + 0] += s0.x; v[8 * j + 1] += s0.y; v[8 * j + 2] += s0.z; v[8 * j + 3] += s0.w;
                v[8 * j + 4] += s1.x; v[8 * j + 5] += s1.y; v[8 * j + 6] += s1.z; v[8 * j + 7] += s1.w;
              }
            } else if (row_ok) {
              for (int src = 0; src < p.ws; ++src) {
                if (src == p.rank) continue;
                const uint8_t* part = p.rs_arena_local + (((size_t)src * p.rs_slot_rows + chunk_row) * p.N[b] + col0) * oes;
                add_row32(part, v, nvalid, o32);
              }
            }
            if (p.reduce_scale != 1.0f) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= p.reduce_scale;
            }
          }
          if (use_tma) {
#pragma unroll
            for (int j = 0; j < 16; ++j) packed[hf][j] = pack16(v[2 * j], v[2 * j + 1], o16h);
          } else if (row_ok) {
            uint8_t* dst;
            if (rs_remote) {
              dst = p.rs_arena_peer[ti.chunk] + (((size_t)p.rank * p.rs_slot_rows + chunk_row) * p.N[b] + col0) * oes;
            } else if (p.mode == MODE_RS) {
              dst = reinterpret_cast<uint8_t*>(p.out[b]) + ((size_t)chunk_row * p.ldo[b] + col0) * oes;
            } else {
              dst = reinterpret_cast<uint8_t*>(p.out[b]) + ((size_t)grow * p.ldo[b] + col0) * oes;
            }
            store_row32(dst, v, nvalid, o32, o16h);
          }
        }
        if (use_tma) {
          if (own_any) __syncwarp();   // every lane has read its sums: the buffer may be reused
          // 16-byte chunk c of this thread's row goes where the 128-byte swizzle expects it
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if ((g * 2 + hf) * 32 >= ti.n_valid) break;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t chunk = (uint32_t)(hf * 4 + j) ^ (uint32_t)(lane & 7);
              ptx::st_shared_v4(stg + lane * ROW_BYTES + chunk * 16, packed[hf][4 * j], packed[hf][4 * j + 1],
                                packed[hf][4 * j + 2], packed[hf][4 * j + 3]);
            }
          }
          ptx::fence_proxy_async_shared();
          if (coop) {
            // The four warps' 4 KiB blocks of this 64-column group are contiguous both in the staging buffer
            // and in the owner's arena: ONE linear 16 KiB bulk copy over NVLink, as it is (swizzled; the owner
            // undoes the swizzle when it reads). Larger copies use the link much better than 4 KiB ones.
            // Before the four warps meet, the leader makes sure that its earlier copies have finished reading
            // shared memory, so that after the barrier the other buffer may be overwritten.
            if (epi_leader) ptx::bulk_wait_group_read<0>();
            ptx::named_bar_sync(2, EPI_WARPS * 32);
            if (epi_leader) {
              const size_t blk = (((size_t)p.rank * sched.tiles_per_chunk + ti.tile_in_chunk) * (BN / 64) + g) * 4;
              ptx::bulk_store(p.rs_arena_peer[ti.chunk] + blk * (32 * ROW_BYTES), stg_all + (stg_count & 1u) * (uint32_t)L::STG_BUF_BYTES,
                              EPI_WARPS * 32 * ROW_BYTES);
              ptx::bulk_commit_group();
            }
          } else {
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(tm_st, stg, ti.n0 + g * 64, st_row);
              ptx::bulk_commit_group();
            }
          }
          note_commit();
          ++stg_count;
        }
      }
      // Release the accumulator to the MMA warp.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(acc), 0)); else ptx::mbar_arrive(tempty_bar(acc));
      }
      if (tracing && epi_leader) trace_put(p, lt, TR_EPI_END_T, globaltimer_ns());

      prev_coop = coop;
      if (p.mode == MODE_RS && own) ++own_seen;
      if (rs_remote) {
        // The owner's flag for this tile is released (two tiles at a time) once the queue of four is full,
        // before this CTA waits on its peers, or after the loop.
        push_pending(p.rs_flag_peer[ti.chunk] + (size_t)p.rank * p.rs_max_tiles + ti.tile_in_chunk, !use_tma);
      }
    }
    publish_pending();
    if (lane == 0) ptx::bulk_wait_group<0>();   // shared memory must outlive the last stores
    __syncwarp();
  } else {
    // ============================================================ communication warps
    if (p.mode == MODE_RS && p.ws > 2 && p.rs_arena_tma != 0) {
      // Reduce-scatter: for every tile of this CTA that the local rank owns, wait for the peers'
      // partials, add them up block by block (coalesced 16-byte loads, two peers in flight per
      // warp) and leave the fp32 sums for the epilogue. This runs while the epilogue warps are
      // still busy sending other ranks' tiles.
      const int cw = warp - (2 + EPI_WARPS);
      const size_t src_stride = (size_t)sched.tiles_per_chunk * (BN / 64) * 4 * (32 * ROW_BYTES);
      uint32_t done = 0;
      uint32_t lt = 0;
      constexpr bool tracing = TRACE;
      for (int t = tile_first; t < sched.total_tiles; t += tile_step, ++lt) {
        const TileInfo ti = decode_tile<BN, PAIR>(p, sched, t, crank);
        if (ti.chunk != p.rank) continue;
        // One thread waits for the peers' flags; its verdict (which also covers an abort raised by
        // another role) goes through shared memory, so that all six warps take the same branch.
        if (cw == 0 && lane == 0) {
          bool ok = true;
          for (int src = 0; src < p.ws && ok; ++src) {
            if (src == p.rank) continue;
            ok = flag_wait<true>(p.rs_flag_local + (size_t)src * p.rs_max_tiles + ti.tile_in_chunk, p.epoch, p,
                                 abort_flag, ST_TIMEOUT_PARTIAL, (uint32_t)src);
          }
          if (*abort_flag) ok = false;
          sum_verdict[done & 1u] = ok ? 1u : 0u;
          if (tracing) trace_put(p, lt, TR_FLAGS_T, globaltimer_ns());
        }
        ptx::named_bar_sync(3, COMM_WARPS * 32);
        if (sum_verdict[done & 1u] == 0u) break;
        const int groups = (ti.n_valid + 63) / 64;
        // Unit of work: half of a 4 KiB block (16 rows x 64 columns), with ALL peers' copies of it loaded
        // before the first add: one memory round trip per unit (the partials come from HBM, they arrived
        // over NVLink), where loading two peers at a time took four.
        for (int unit = cw; unit < groups * 8; unit += COMM_WARPS) {
          const int blk16 = unit >> 1, half = unit & 1;
          const size_t blk = ((size_t)ti.tile_in_chunk * (BN / 64) * 4 + blk16);
          const uint8_t* base = p.rs_arena_local + blk * (32 * ROW_BYTES) + half * (16 * ROW_BYTES);
          uint4 q[MAX_WORLD - 1][4];
#pragma unroll
          for (int u = 0; u < MAX_WORLD - 1; ++u) {
            if (u < p.ws - 1) {
              const uint8_t* bp = base + (size_t)((p.rank + 1 + u) % p.ws) * src_stride;
#pragma unroll
              for (int i = 0; i < 4; ++i) q[u][i] = ptx::ld_cg_v4(bp + (size_t)(i * 32 + lane) * 16);
            }
          }
          float sum[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[j] = 0.0f;
#pragma unroll
          for (int u = 0; u < MAX_WORLD - 1; ++u) {
            if (u < p.ws - 1) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t w[4] = {q[u][i].x, q[u][i].y, q[u][i].z, q[u][i].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  sum[8 * i + 2 * e] += __uint_as_float(w[e] << 16);
                  sum[8 * i + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
                }
              }
            }
          }
          // chunk L = half*128 + i*32 + lane of the bf16 block becomes units 2L and 2L+1 of the 8 KiB fp32 block
          float4* op = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p.rs_sum_local) + blk * (size_t)(64 * ROW_BYTES));
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int Lc = half * 128 + i * 32 + lane;
            op[2 * Lc] = make_float4(sum[8 * i], sum[8 * i + 1], sum[8 * i + 2], sum[8 * i + 3]);
            op[2 * Lc + 1] = make_float4(sum[8 * i + 4], sum[8 * i + 5], sum[8 * i + 6], sum[8 * i + 7]);
          }
        }
        __threadfence();
        ptx::named_bar_sync(3, COMM_WARPS * 32);
        ++done;
        if (cw == 0 && lane == 0) {
          *sums_done = done;
          if (tracing) trace_put(p, lt, TR_SUMS_T, globaltimer_ns());
        }
      }
    }
    if (p.mode == MODE_AG) {
      const int cw = warp - (2 + EPI_WARPS);
      const int gw = blockIdx.x * COMM_WARPS + cw;
      const int total_warps = gridDim.x * COMM_WARPS;
      const int full_pieces = ag_tile_pieces(p, 0);
      const int total_pieces = (int)((p.ag_chunk_bytes + PIECE_BYTES - 1) / PIECE_BYTES);  // flat, staging only
      // ---- step 0: stage the local shard for the peers (and in the gathered buffer if asked).
      const bool stage_symm = p.ws > 1;
      if (stage_symm || p.ag_copy_own) {
        uint8_t* dst_a = stage_symm ? p.ag_symm_local : p.ag_gathered + (size_t)p.rank * p.ag_chunk_bytes;
        uint8_t* dst_b = (stage_symm && p.ag_copy_own) ? p.ag_gathered + (size_t)p.rank * p.ag_chunk_bytes : nullptr;
        for (int q = gw; q < total_pieces; q += total_warps) {
          const long long off = (long long)q * PIECE_BYTES;
          const int n16 = (int)(min((long long)PIECE_BYTES, p.ag_chunk_bytes - off) >> 4);
          copy_piece(p.ag_src + off, dst_a + off, dst_b ? dst_b + off : nullptr, n16, lane);
        }
        if (p.ag_has_scale && stage_symm) {
          float* sdst = reinterpret_cast<float*>(p.ag_symm_local + p.ag_scale_off);
          for (int i = gw * 32 + lane; i < p.rows_per_rank; i += total_warps * 32) sdst[i] = __ldg(p.ag_scale_src + i);
        }
      }
      if (stage_symm) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const uint32_t prev = atomicAdd(p.ctrl, 1u);
          if (prev == (uint32_t)total_warps - 1u) {
            __threadfence_system();
            for (int r = 0; r < p.ws; ++r) {
              if (r != p.rank) ptx::st_release_sys(p.staged_peer[r] + p.rank * FLAG_STRIDE, p.epoch);
            }
          }
        }
        __syncwarp();
      }
      // ---- pull the peers' shards. Piece q of the schedule comes from peer rank+1+(q % (ws-1)), so
      //      consecutive warps read from different peers and every row block of every peer fills
      //      at the same pace (the order the tile schedule consumes them in).
      if (p.ws > 1) {
        const int npeers = p.ws - 1;
        const long long tile_bytes = (long long)BM * p.K * p.elem_bytes;
        uint32_t seen = 0;   // peers whose "staged" flag this warp has acquired
        bool ok = true;
        auto acquire_peer = [&](int src) -> bool {
          if (seen & (1u << src)) return true;
          bool good = true;
          if (lane == 0) {
            good = flag_wait<true>(p.staged_local + src * FLAG_STRIDE, p.epoch, p, abort_flag, ST_TIMEOUT_STAGED, (uint32_t)src);
          }
          good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;
          seen |= (1u << src);
          return good;
        };
        if (p.ag_has_scale) {
          const int units = sched.mt_per_chunk * npeers;
          for (int v = gw; v < units && ok; v += total_warps) {
            const int src = (p.rank + 1 + v % npeers) % p.ws;
            const int mt = v / npeers;
            ok = acquire_peer(src);
            if (!ok) break;
            const float* ps = reinterpret_cast<const float*>(p.ag_symm_peer[src] + p.ag_scale_off);
            float* gs = p.ag_scale_gathered + (size_t)src * p.rows_per_rank;
            const int rows = min(BM, p.rows_per_rank - mt * BM);
            for (int i = lane; i < rows; i += 32) {
              uint32_t w;
              asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(w) : "l"(ps + mt * BM + i) : "memory");
              gs[mt * BM + i] = __uint_as_float(w);
            }
            __threadfence();
            __syncwarp();
            if (lane == 0) ptx::red_add_release_gpu(p.ready + src * sched.mt_per_chunk + mt, 1u);
          }
        }
        // Software pipeline: the loads of piece i are in flight while piece i-1 (stored in the
        // previous iteration) is fenced and published.
        const long long total_q = (long long)sched.mt_per_chunk * full_pieces * npeers;
        uint32_t* prev_ready = nullptr;
        for (long long q = gw; q < total_q && ok; q += total_warps) {
          const int src = (p.rank + 1 + (int)(q % npeers)) % p.ws;
          const long long qq = q / npeers;
          const int mt = (int)(qq / full_pieces);
          const int j = (int)(qq - (long long)mt * full_pieces);
          const long long tile_start = (long long)mt * tile_bytes;
          const long long tile_end = min(tile_start + tile_bytes, (long long)p.ag_chunk_bytes);
          const long long off = tile_start + (long long)j * PIECE_BYTES;
          if (off >= tile_end) continue;   // the last row block of a chunk may have fewer pieces
          ok = acquire_peer(src);
          if (!ok) break;
          const uint8_t* peer = p.ag_symm_peer[src];
          uint8_t* dst = p.ag_gathered + (size_t)src * p.ag_chunk_bytes;
          const int n16 = (int)(min((long long)PIECE_BYTES, tile_end - off) >> 4);
          uint4 r[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = u * 32 + lane;
            if (i < n16) r[u] = ptx::ld_relaxed_sys_v4(peer + off + (size_t)i * 16);
          }
          if (prev_ready != nullptr) {
            ptx::fence_proxy_async_global();
            __threadfence();
            __syncwarp();
            if (lane == 0) ptx::red_add_release_gpu(prev_ready, 1u);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = u * 32 + lane;
            if (i < n16) reinterpret_cast<uint4*>(dst + off)[i] = r[u];
          }
          prev_ready = p.ready + src * sched.mt_per_chunk + mt;
        }
        if (prev_ready != nullptr) {
          ptx::fence_proxy_async_global();
          __threadfence();
          __syncwarp();
          if (lane == 0) ptx::red_add_release_gpu(prev_ready, 1u);
        }
      }
    }
  }

  // ============================================================ teardown
  ptx::tc_fence_before();
  if (PAIR) ptx::cluster_sync(); else __syncthreads();   // pair: nobody signals a CTA that has left
  if (TRACE && threadIdx.x == 0) {
    trace_put(p, 0, TR_CTA_END_T, globaltimer_ns());
    trace_put(p, 1, TR_CTA_END_T, (unsigned long long)clock64());
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS); else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace apk
