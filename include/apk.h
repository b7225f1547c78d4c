/*
 * apk.h - C ABI of libapk.so, the sm_100a (B200) implementation of AutoParallel's async
 * tensor-parallel hot path: all-gather -> matmul and matmul -> reduce-scatter, bf16 and fp8
 * (e4m3, row-wise scales), with the communication done inside the GEMM kernel over NVLink
 * peer mappings.
 *
 * The library takes plain device pointers, sizes and a CUDA stream handle; it knows nothing
 * about torch. Every function returns 0 on success or a negative code; apk_last_error()
 * gives the message of the calling thread's last failure. Nothing here falls back to the
 * CPU: on a machine without an sm_100 GPU the op entry points fail with APK_ERR_CUDA.
 *
 * Reference interfaces replaced (paths inside the AutoParallel source tree):
 *   apk_ag_gemm            autoparallel/asynctp_ops.py:395-530  _fused_all_gather_matmul_impl
 *                          + :34-177 _pipelined_multi_all_gather_and_consume, as called by
 *                          the CUDA bodies of fused_all_gather_matmul (:703-752) and
 *                          fused_all_gather_scaled_matmul (:947-1025)
 *   apk_gemm_rs            autoparallel/asynctp_ops.py:1103-1185 _fused_matmul_reduce_scatter_impl,
 *                          :1293-1423 _fused_scaled_matmul_reduce_scatter_impl and
 *                          :209-323 _pipelined_produce_and_all2all
 *   apk_symm_*             the parts of torch's symmetric memory the path uses through
 *                          get_symm_mem_workspace / get_buffer / barrier
 *                          (autoparallel/asynctp_ops.py:61-65, :89-94, :229-242)
 */
#ifndef APK_H_
#define APK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define APK_ABI_VERSION 1
#define APK_MAX_B 4      /* weight matrices that may share one gathered A */
#define APK_MAX_WORLD 8  /* ranks of one tensor-parallel group (one NVSwitch domain) */

enum {
  APK_OK = 0,
  APK_ERR_ARG = -1,     /* bad argument (shape, alignment, dtype, null pointer) */
  APK_ERR_CUDA = -2,    /* a CUDA runtime or driver call failed */
  APK_ERR_SIZE = -3,    /* a workspace, flag pad or fixed scratch area is too small */
  APK_ERR_TIMEOUT = -4, /* a device-side wait ran out (reported by apk_check_status) */
};

enum { APK_BF16 = 0, APK_E4M3 = 1, APK_F32 = 2, APK_F16 = 3 };

/* How a scale operand is laid out. */
enum {
  APK_SCALE_NONE = 0,
  APK_SCALE_SCALAR = 1,        /* one fp32 */
  APK_SCALE_VECTOR = 2,        /* A: one fp32 per row of the local operand; B: one per column */
  APK_SCALE_ROWS_REPLICATED = 3 /* A of an all-gather: one fp32 per row of the gathered A */
};

enum { APK_REDUCE_SUM = 0, APK_REDUCE_AVG = 1 };

/*
 * One tensor-parallel group as seen from this process. data[r] / flags[r] are rank r's
 * symmetric data arena and signal pad mapped into this process (entry [rank] is the local
 * allocation); they come from apk_symm_alloc / apk_symm_import and have the same size on
 * every rank. The data arena is used in two halves that alternate with the parity of
 * `epoch`, which the caller increments by one for every collective call on the group (all
 * ranks call in the same order, so they agree on it). With world == 1, data and flags may
 * be null.
 *
 * Replaces what the reference gets from get_symm_mem_workspace(group_name, size)
 * (autoparallel/asynctp_ops.py:61, :229) plus symm_mem.barrier(channel) (:65, :147, :177,
 * :233, :311-323): there are no separate barrier kernels, the fused kernel releases and
 * acquires per-chunk flags itself.
 */
typedef struct {
  int32_t rank;
  int32_t world;
  void* data[APK_MAX_WORLD];
  void* flags[APK_MAX_WORLD];
  uint64_t data_bytes;  /* size of each data arena (both halves together) */
  uint64_t flag_bytes;  /* size of each signal pad: 4096 bytes of per-rank flags, then world x T per-tile flags
                           (u32); at least 8192, T limits the tiles of one reduce-scatter chunk */
  void* ctrl;           /* local device scratch for per-call counters */
  uint64_t ctrl_bytes;
  uint32_t* status;     /* local device word; 0 while no device wait has timed out */
  uint32_t epoch;
  uint32_t reserved;
  double timeout_s;     /* budget of every device-side wait */
} apk_comm;

/* One right-hand operand and its output. B is [K, N]. */
typedef struct {
  const void* B;
  int64_t ldb;           /* elements between rows (n_major) or between columns (k-contiguous) */
  int32_t n_major;       /* 1: row-major [K][N]; 0: column-major, K contiguous (B = W^T view) */
  int32_t N;
  void* out;             /* AG: [world*rows_per_rank, N]; RS: [M/world, N] */
  int64_t ldo;
  int32_t out_dtype;     /* APK_BF16, APK_F16 or APK_F32 (apk_gemm_rs with peers: not APK_F16, the partials travel as bf16 or f32) */
  int32_t b_scale_mode;  /* APK_SCALE_NONE / SCALAR / VECTOR (per column) */
  const float* b_scale;
  const void* bias;      /* per column, or null */
  int32_t bias_dtype;    /* APK_BF16 or APK_F32 */
  int32_t reserved;
  const float* result_scale; /* one fp32 or null */
} apk_operand;

/*
 * outs[b] = all_gather(A_shard) @ Bs[b], rows ordered by source rank.
 * Mirrors _fused_all_gather_matmul_impl (autoparallel/asynctp_ops.py:395-530) after it has
 * moved gather_dim to the front and flattened A to 2-D (:437-443).
 */
typedef struct {
  int32_t dtype;          /* APK_BF16, APK_F16 or APK_E4M3: element type of A and every B */
  int32_t rows_per_rank;  /* rows of A_shard */
  int32_t K;
  int32_t nB;
  const void* A_shard;    /* [rows_per_rank, K], row-major with lda */
  int64_t lda;
  apk_operand Bs[APK_MAX_B];
  void* A_gathered;       /* [world*rows_per_rank, K] contiguous. Required when world > 1 or return_A. */
  int32_t return_A;       /* also place the local shard in A_gathered */
  int32_t a_scale_mode;   /* NONE / SCALAR / VECTOR (row-wise, sharded like A) / ROWS_REPLICATED */
  const float* A_scale;
  float* A_scale_gathered; /* [world*rows_per_rank] scratch, required for VECTOR when world > 1 */
  int32_t gather_k;       /* 0: shards are row blocks of A (rows ordered by rank). 1: shards are K-slices
                             [rows_per_rank, K] of A [rows_per_rank, world*K]; every B is [world*K, N],
                             outs[b] is [rows_per_rank, N], A_gathered is [world][rows_per_rank][K]
                             (autoparallel/asynctp_ops.py:602-669). bf16, no scales. */
  int32_t reserved;
} apk_ag_gemm_args;

/*
 * out = reduce_scatter(A @ B) along rows: rank d receives rows [d*M/world, (d+1)*M/world)
 * summed (or averaged) over ranks. Mirrors _fused_matmul_reduce_scatter_impl
 * (autoparallel/asynctp_ops.py:1159-1185) after scatter_dim was moved to the front.
 */
typedef struct {
  int32_t dtype;
  int32_t M;              /* rows of A; divisible by world */
  int32_t K;
  int32_t reduce_op;      /* APK_REDUCE_SUM / APK_REDUCE_AVG */
  const void* A;          /* [M, K] row-major with lda */
  int64_t lda;
  apk_operand B;          /* B.out is [M/world, N] */
  int32_t a_scale_mode;   /* NONE / SCALAR / VECTOR (one per row of A) */
  int32_t scatter_cols;   /* 0: rank d receives rows [d*M/world, ...). 1: rank d receives columns
                             [d*N/world, ...) of all M rows: B.N is the FULL width, B.out is [M, N/world]
                             (autoparallel/asynctp_ops.py:1129-1157). No scales. */
  const float* A_scale;
} apk_gemm_rs_args;

int apk_abi_version(void);
const char* apk_last_error(void);

/* ---- symmetric memory: cudaMalloc + CUDA IPC handles (one process per GPU). ---- */
int apk_symm_alloc(uint64_t bytes, void** ptr);             /* zero-filled, on the current device */
int apk_symm_free(void* ptr);
int apk_symm_export(const void* ptr, uint8_t handle[64]);   /* handle to ship to the peers */
int apk_symm_import(const uint8_t handle[64], void** ptr);  /* map a peer's allocation */
int apk_symm_unimport(void* ptr);

/* Bytes the ops need in each HALF of the data arena / in ctrl / tiles of the flag pad. */
uint64_t apk_ag_gemm_arena_bytes(const apk_ag_gemm_args* args, int32_t world);
uint64_t apk_gemm_rs_arena_bytes(const apk_gemm_rs_args* args, int32_t world);
uint64_t apk_ctrl_bytes(int32_t rows_per_rank, int32_t world);

/* ---- ops: enqueue on `stream` (a cudaStream_t) of the current device and return. ---- */
int apk_ag_gemm(const apk_comm* comm, const apk_ag_gemm_args* args, void* stream);
int apk_gemm_rs(const apk_comm* comm, const apk_gemm_rs_args* args, void* stream);

/*
 * Stand-alone collectives over the same arena, signal pad and epoch (each call is one collective:
 * increment comm->epoch). out = every rank's shard, ordered by rank; every shard has shard_bytes
 * (a multiple of 16). Replaces _low_contention_all_gather (autoparallel/asynctp_ops.py:1524-1610).
 */
int apk_all_gather(const apk_comm* comm, const void* shard, void* out, uint64_t shard_bytes, void* stream);
/*
 * `in` holds world parts of out_bytes each; out = sum (or mean) over ranks of part [rank]. Elements are
 * bf16 or fp32, accumulated in fp32. Replaces _low_contention_reduce_scatter (:1613-1702).
 */
int apk_reduce_scatter(const apk_comm* comm, const void* in, void* out, uint64_t out_bytes, int32_t dtype,
                       int32_t reduce_op, void* stream);

/*
 * apk_ag_gemm without caller-provided scratch. It has no counterpart in the reference.
 *
 * For callers that cannot allocate device memory around the op: a serving runtime that has
 * already handed the whole GPU to its own pool (a cudaMalloc there fails or eats into the
 * pool's headroom), or code on a path where allocating is forbidden because cudaMalloc may
 * synchronise the device. Inputs and outputs are passed as for apk_ag_gemm; comm->status stays
 * the caller's word, because the caller reads it. The scratch apk_ag_gemm takes from its caller
 * is ignored and comes from one fixed device array inside the library instead:
 *   comm->ctrl / ctrl_bytes   per-call counters, up to 64 KiB
 *   args->A_gathered          only when return_A == 0: up to 32 MiB (world * rows_per_rank * K * element size)
 *   args->A_scale_gathered    up to 65536 gathered rows
 * A call that needs more returns APK_ERR_SIZE and launches nothing. The function calls no
 * cudaMalloc / cudaFree. The first call on a device looks up the array's address and sets the
 * kernel's shared-memory attribute, so make that first call outside any stream capture.
 * Every call on a GPU uses the same array (it keeps the previous call's contents; the counters
 * are cleared per call): calls that may overlap on the GPU, e.g. on two streams, race.
 * Each GPU that loads the library holds the 32.3 MiB array until the process exits.
 */
int apk_ag_gemm_static(const apk_comm* comm, const apk_ag_gemm_args* args, void* stream);

/* Synchronises `stream`, reads the status word, clears it; APK_ERR_TIMEOUT if it was set. */
int apk_check_status(const apk_comm* comm, void* stream, uint32_t* raw);

/*
 * Test utility, no GPU needed: the order in which the persistent kernel's CTAs (pair = 0) or CTA pairs
 * (pair = 1, crank = rank inside the pair) enumerate the tiles of a problem, computed with the kernel's
 * own scheduling functions. mode: 0 plain, 1 all-gather, 2 reduce-scatter; last_dim: the K-split /
 * column-split variants. Writes up to `capacity` rows of 6 ints (chunk, row block, operand, first
 * column, tile index inside the chunk, valid rows) and returns the number of scheduling units.
 */
int apk_debug_schedule(int32_t mode, int32_t world, int32_t rank, int32_t rows_per_rank, int32_t nB, const int32_t* N,
                       int32_t last_dim, int32_t pair, int32_t crank, int32_t* out, int32_t capacity);

/* Test utility: the reduce-scatter lag (row blocks between the peers' row block j and the own one) that
 * apk_debug_schedule uses from now on; 0 = the built-in default. Real launches compute theirs from the grid. */
void apk_debug_set_rs_lag(int32_t row_blocks);

/* Kernels launched by this library in this process so far (memsets not counted). */
uint64_t apk_launch_count(void);
/* ... of which launched as clusters of two CTAs (tcgen05 cta_group::2). */
uint64_t apk_pair_launch_count(void);
/* Calls whose shape qualified for CTA pairs but ran on single CTAs because the device cannot schedule
 * clusters of two (the reason is in apk_last_error() of the first such call). 0 on a healthy B200. */
uint64_t apk_pair_refusal_count(void);

/*
 * Timeline of the fused kernel, for profiling (the reference wraps each op in
 * torch.profiler.record_function, autoparallel/asynctp_ops.py:741, :1077; a single kernel needs
 * stamps from inside). While `buf` (device memory of the current device, zero-filled by the
 * caller, `bytes` long) is set, every apk_ag_gemm / apk_gemm_rs launch on that device whose
 * records fit writes 16 u64 per (CTA, local tile): record index = blockIdx * tiles_per_cta +
 * local tile, tiles_per_cta = ceil(scheduling units / scheduled CTAs or CTA pairs). Fields, in
 * order: tile index + 1; first load issued (ns, %globaltimer); producer cycles waiting for
 * gathered rows; for free stages; first MMA issued (ns); MMA-thread cycles waiting for
 * operands; for a free accumulator; last MMA committed (ns); accumulator complete (ns);
 * epilogue cycles waiting for peers' partials; epilogue done (ns); cycles spent publishing
 * flags; peers' flags of an own tile acquired (ns); their sums written (ns); CTA begin and
 * end (ns, record 0 of each CTA only). Pass null to switch it off. Not thread-safe against
 * concurrent launches; costs one predictable branch per stamp when off.
 */
int apk_set_trace(void* buf, uint64_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* APK_H_ */
