/*
 * sparseflow_b200 -- C ABI of the Blackwell (sm_100a) 2:4-sparse FFN path.
 *
 * Plain C, plain pointers and sizes.  Unless a function says otherwise every data pointer is a
 * DEVICE pointer, every call is asynchronous on the given CUDA stream (`stream` is a cudaStream_t
 * passed as void*, NULL = default stream) and returns an sfb200_status.  There is no CPU fallback:
 * without a usable sm_100 device the compute entry points return SFB200_ERROR_CUDA.
 *
 * Three groups of entry points:
 *   1. sfb200_*       the hot path itself (prune+compress, sparse GEMM, gated FFN)
 *   2. sf_*           the reference's runtime selection API, same structs and semantics
 *   3. sparseflow_*   the reference's "stable C ABI v1", whose compute calls are stubs upstream
 *
 * Each declaration cites the reference interface it stands in for (path:line in the reference
 * tree).
 */
#ifndef SPARSEFLOW_B200_H
#define SPARSEFLOW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SFB200_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ common ---------------- */

typedef enum {
  SFB200_SUCCESS = 0,
  SFB200_ERROR_INVALID_ARGUMENT = 1,
  SFB200_ERROR_OUT_OF_MEMORY = 2,
  SFB200_ERROR_CUDA = 3,
  SFB200_ERROR_NOT_SUPPORTED = 4,
  SFB200_ERROR_TENSOR_MAP = 8,
  SFB200_ERROR_DEVICE = 9, /* a kernel gave up on a bounded wait; see sfb200_device_status */
  SFB200_ERROR_SCRATCH_TOO_SMALL = 10 /* sfb200_ffn_forward_noalloc: hidden tensor exceeds the static scratch */
} sfb200_status;

typedef enum { SFB200_F16 = 0, SFB200_BF16 = 1 } sfb200_dtype;
/* which element wins a magnitude tie inside a group of four */
typedef enum { SFB200_TIE_HIGH = 0 /* reference behaviour */, SFB200_TIE_LOW = 1 } sfb200_tie;
typedef enum { SFB200_ACT_NONE = 0, SFB200_ACT_RELU = 1, SFB200_ACT_SILU = 2, SFB200_ACT_GELU = 3 } sfb200_act;

SFB200_API const char* sfb200_status_string(int status);
SFB200_API int sfb200_version(void); /* major*10000 + minor*100 + patch */

/* Bytes of the compressed-values buffer ([rows, K/2] 16-bit) and of the tiled metadata buffer
 * (128x128 tiles of 2 KiB, rows and K rounded up to 128) for a rows x K weight. */
SFB200_API size_t sfb200_values_bytes(int rows, int K);
SFB200_API size_t sfb200_meta_bytes(int rows, int K);

/* Synchronise the current device and return the device status word (0 = ok) of the kernels
 * launched so far; the word is cleared.  Non-zero: (code << 8) | detail, code 1 = a bounded
 * mbarrier wait ran out (detail = which wait: 1 operand slot free, 2 operands landed, 3 accumulator
 * free, 4 accumulator complete).  Returns SFB200_ERROR_DEVICE when the word was non-zero.  Includes
 * the word of sfb200_ffn_forward_noalloc (see sfb200_noalloc_device_status).  May allocate the
 * per-device state on first use.  Plays the role of upstream's failure report that feeds the
 * quarantine (runtime/dispatch/eligibility_policy.cpp:72-84): callers pass a non-zero result on
 * to sf_record_sparse_failure. */
SFB200_API int sfb200_device_status(int* status_word);

/* Test hook for that failure path (no counterpart upstream): launches one small CTA that waits, with
 * a limit of `limit_us` microseconds (1 .. 100000), on a barrier nothing arrives on.  The wait gives
 * up, the kernel records (1 << 8) | where in the status word (the regular one, or the one of the
 * allocation-free entry point when noalloc_word != 0) and returns by itself; nothing faults or traps
 * and the context stays usable.  0 <= where <= 255. */
SFB200_API int sfb200_debug_wait_timeout(unsigned limit_us, int where, int noalloc_word, void* stream);

/* ------------------------------------------------------------------ 1. hot path ----------- */

/*
 * 2:4 magnitude prune + compress of dense[rows, K] (row pitch ld elements).
 * Stands in for experiments/prune_24_cpu.py:17-28 (selection rule, values, code bytes),
 * sparseflow/nn/sparseflow_linear.py:20-35 (prune_24_dense_weight) and the
 * torch.sparse.to_sparse_semi_structured call sites sparseflow/fused_mlp.py:22,28,
 * sparseflow/nn/sparseflow_linear.py:66, sparseflow/nn/sparseflow_mlp.py:62-76.
 * Any of the four outputs may be NULL.  `meta` needs K % 16 == 0 and 16-byte aligned buffers.
 *   values    [rows, K/2]   kept pair per group, index order
 *   meta      sfb200_meta_bytes(rows, K) bytes, layout consumed by sfb200_sparse_gemm
 *   ref_codes [rows, K/4]   uint8, the reference script's PAIR_TO_CODE byte per group
 *   pruned    [rows, K]     pruned dense copy
 */
SFB200_API int sfb200_prune_compress_24(const void* dense, int rows, int K, int ld, int dtype,
                                        int tie, void* values, void* meta, void* ref_codes,
                                        void* pruned, void* stream);

/*
 * Same, for the fused gate|up weight of the gated FFN: reads gate[I, K] and up[I, K] and emits
 * the 2*I-row matrix whose rows alternate in blocks of 16 (16 gate rows, the matching 16 up
 * rows, ...), which is the row order sfb200_sparse_gemm_swiglu expects.  Replaces the
 * torch.cat([gate, up]) + to_sparse_semi_structured of sparseflow/fused_mlp.py:16-24.
 * I % 16 == 0.
 */
SFB200_API int sfb200_prune_compress_gate_up(const void* gate, const void* up, int I, int K, int ld,
                                             int dtype, int tie, void* values, void* meta,
                                             void* stream);

/* is_valid_dev (device int) := 1 iff every group of four has <= 2 non-zeros.
 * Device-pointer form of sparseflow_validate_2_4 (include/sparseflow/c_api.h:171-176). */
SFB200_API int sfb200_validate_24(const void* w, int rows, int K, int ld, int* is_valid_dev,
                                  void* stream);

/* values + meta -> pruned dense [rows, K] (row pitch ld). */
SFB200_API int sfb200_decompress_24(const void* values, const void* meta, int rows, int K,
                                    void* dense, int ld, void* stream);

/*
 * Y[M, N] = act(X[M, K] . W[N, K]^T + bias), W given as (values, meta).  fp32 accumulate,
 * output in `dtype`.  ldx / ldy are row pitches in elements.  K % 64 == 0, N % 8 == 0.
 * Stands in for aten::_sparse_semi_structured_mm / torch.mm(x, Wsp.t()) / F.linear(x, Wsp) at
 * sparseflow/nn/sparseflow_linear.py:123, sparseflow/nn/sparseflow_mlp.py:95,97,
 * sparseflow/fused_mlp.py:54,60, and for sparseflow_sparse_gemm (c_api.h:151-160).
 */
SFB200_API int sfb200_sparse_gemm(const void* x, int ldx, const void* values, const void* meta,
                                  void* y, int ldy, int M, int N, int K, int dtype,
                                  const void* bias, int act, void* stream);

/* Same with FLOAT output y[M, N] (row pitch ldy floats): the fp32 accumulators (+ bias, activation) are stored
 * unrounded.  For the partial sums of a row-parallel GEMM, whose rounding to 16 bits should happen once, after
 * the sum over ranks.  Prefill kernel only (any M; small M runs it on one tile).  No counterpart upstream. */
SFB200_API int sfb200_sparse_gemm_f32out(const void* x, int ldx, const void* values, const void* meta, float* y,
                                         int ldy, int M, int N, int K, int dtype, const void* bias, int act,
                                         void* stream);

/*
 * H[M, I] = silu(X . Wg^T) * (X . Wu^T) with the fused gate|up weight produced by
 * sfb200_prune_compress_gate_up (2*I rows).  One GEMM, SiLU.mul in the epilogue: replaces the
 * fused GEMM + chunk + act*up of sparseflow/fused_mlp.py:77-83 and the Triton kernel
 * sparseflow/kernels/fused_silu_mul.py:6-31.
 */
SFB200_API int sfb200_sparse_gemm_swiglu(const void* x, int ldx, const void* values_gu,
                                         const void* meta_gu, void* h, int ldh, int M, int I, int K,
                                         int dtype, void* stream);

/* out[r, c] = silu(gate[r, c]) * up[r, c], fp32 math (sparseflow/kernels/fused_silu_mul.py:33-57).
 * Unfused variant, kept for the dense branch of the shape gate. */
SFB200_API int sfb200_silu_mul(const void* gate, int ld_gate, const void* up, int ld_up, void* out,
                               int ld_out, int rows, int cols, int dtype, void* stream);

/*
 * Gated FFN forward, out[M, H] = down(silu(gate(x)) * up(x)) (+ down_bias):
 * sparseflow/fused_mlp.py:63-98 (SparseFlowFusedMLP.forward) with both GEMMs sparse.
 * `hidden` is caller-provided scratch of M * I elements.
 */
typedef struct {
  int H;                 /* hidden size   (K of gate/up, N of down) */
  int I;                 /* intermediate  (N of gate/up, K of down) */
  int dtype;             /* sfb200_dtype */
  const void* gu_values; /* fused gate|up weight, 2*I rows x H      */
  const void* gu_meta;
  const void* down_values; /* down weight, H rows x I               */
  const void* down_meta;
  const void* down_bias; /* [H] or NULL */
} sfb200_ffn_weights;

SFB200_API int sfb200_ffn_forward(const sfb200_ffn_weights* w, const void* x, int ldx, void* hidden,
                                  void* out, int ldo, int M, void* stream);

/*
 * Same with HOST input and output buffers (pinned memory recommended): copies x to the device,
 * runs the FFN, copies the result back, and synchronises the stream.  Device staging buffers are
 * owned by the library, grown on demand and reused.  This is the call a host-side integration
 * without its own device buffers makes.
 */
SFB200_API int sfb200_ffn_forward_host(const sfb200_ffn_weights* w, const void* x_host,
                                       void* out_host, int M, void* stream);

/*
 * Tensor-parallel building blocks (no counterpart in the reference, which has no distributed code).  One process per
 * GPU; buffers that other ranks touch live in peer-mapped memory (e.g. torch symmetric memory).  The FFN shards as
 * column-parallel gate/up and row-parallel down; the row-parallel GEMM leaves partial sums that must be added across
 * ranks (reduce-scatter) and the finished token blocks replicated (all-gather).
 *
 * Row-parallel GEMM with the reduce-scatter fused into its epilogue: rank r computes its partial
 * Y_r[M, N] = X_r . W_r^T and stores token block o (tok_per_owner tokens, a multiple of 16) straight into
 * peer_slots[o], rank o's receive slot for rank r ([tok_per_owner, N]), with plain stores over NVLink that overlap the
 * GEMM tile by tile.  peer_slots is a HOST array of tp device pointers.  tp <= 8.  `rank` is the caller's rank: its
 * token tiles are visited starting at rank + 1's block, so that the ranks write to different owners at any one time
 * instead of all to the same one.  slots_f32 selects the element type
 * of the slots, here and in the reduction calls below: 0 = `dtype`; 1 = float (the partial sums are rounded to 16 bits
 * only once, after they have been added); 2 = fp16 whatever `dtype` is, clamped to +-65504 (half the bytes of float on
 * the wire, 11 significant bits instead of bf16's 8: measured inside the single-GPU error bound where bf16 slots are not).
 */
SFB200_API int sfb200_sparse_gemm_scatter(const void* x, int ldx, const void* values, const void* meta,
                                          void* const* peer_slots, int tp, int rank, int tok_per_owner, int slots_f32, int M,
                                          int N, int K, int dtype, void* stream);
/*
 * Second half, ONE launch per rank with the cross-GPU ordering inside the kernel: waits until every rank's GEMM has
 * finished (flag words in symmetric memory, bounded polls), adds the first `rows` rows of the tp local receive slots
 * slots[tp][slot_rows, cols] in fp32, adds the bias, rounds once, stores the finished block into every rank's
 * output -- peer_out_blocks[d] = this rank's token block inside rank d's output tensor (plain 16-byte peer stores), or
 * mc_out_block when the output has a switch-replicated mapping (one multimem.st) -- and returns once every rank has
 * finished, so the next step may overwrite the slots.
 *   peer_flags  HOST array of tp device pointers: every rank's flag array (sfb200_tp_flag_words() uint32, zero before
 *               the first launch, symmetric memory, used by no one else)
 *   epoch       1, 2, 3, ...: one per launch on these flags, the same on every rank
 * Every rank must make the same sequence of calls.  A peer that never arrives makes the wait give up after 2 s:
 * sfb200_device_status then reports (2 << 8) | phase and the output is not valid.
 */
SFB200_API int sfb200_tp_reduce_slots(const void* slots, int slot_rows, int slots_f32, void* mc_out_block,
                                      void* const* peer_out_blocks, int rows, int cols, int dtype, const void* bias,
                                      void* const* peer_flags, int tp, int rank, unsigned epoch, void* stream);
/*
 * The whole exchange of one token chunk in ONE launch, for a GEMM that wrote its partial sums LOCALLY
 * (sfb200_sparse_gemm / sfb200_sparse_gemm_f32out into partial_chunk): push phase -- owner block o of the chunk
 * ([tp][block_rows, cols], valid_rows[o] live rows) is copied to peer_slots[o], the slot rank o keeps for this rank --
 * then sfb200_tp_reduce_slots on this rank's own slots.  light = 1 launches a 128-thread form that fits beside a GEMM
 * CTA on every SM, so that on a side stream the exchange of chunk c runs while the GEMMs of chunk c + 1 do.
 */
SFB200_API int sfb200_tp_push_reduce(const void* partial_chunk, int block_rows, const int* valid_rows,
                                     void* const* peer_slots, const void* slots, int slot_rows, int slots_f32,
                                     void* const* peer_out_blocks, int rows, int cols, int dtype, const void* bias,
                                     void* const* peer_flags, int tp, int rank, unsigned epoch, int light,
                                     void* stream);
/*
 * The same exchange pulled through NVSwitch instead: every rank has written its partial output (sfb200_sparse_gemm or
 * sfb200_sparse_gemm_f32out) into its own copy of a symmetric buffer that has a switch-replicated ("multicast")
 * mapping; this rank's token block is summed across ranks inside the switch (multimem.ld_reduce) and the finished
 * block written to every rank (multimem.st).  Same flags / epoch protocol.
 *   mc_partial_block  this rank's token block ([rows, cols]) inside the MULTICAST mapping of the partial buffer;
 *                     partial_f32 = 1: FLOAT partials, summed in fp32, output rounded once; partial_f32 = 0: 16-bit
 *                     partials (half the bytes; every rank's partial carries its own 16-bit rounding)
 *   mc_out_block      the same block inside the multicast mapping of the output tensor
 */
SFB200_API int sfb200_tp_allreduce_switch(const void* mc_partial_block, void* mc_out_block, int rows, int cols,
                                          int dtype, int partial_f32, const void* bias, void* const* peer_flags,
                                          int tp, int rank, unsigned epoch, void* stream);
/* Same protocol, no reduction: local_block ([rows, cols] 16-bit, LOCAL memory) is copied into every rank's buffer:
 * mc_dst_block (multimem.st) when non-NULL, else peer_dst_blocks[d] (peer stores).  An all-gather of one block per
 * rank, e.g. of the activations each rank uploaded. */
SFB200_API int sfb200_tp_allgather(const void* local_block, void* mc_dst_block, void* const* peer_dst_blocks, int rows,
                                   int cols, void* const* peer_flags, int tp, int rank, unsigned epoch, void* stream);
SFB200_API int sfb200_tp_flag_words(void);
/*
 * Gated FFN forward for callers that cannot allocate device memory (no counterpart in the
 * reference).  Same computation and bits as sfb200_ffn_forward, but the M x I hidden tensor lives
 * in a fixed array inside the library image, so this call and everything under it performs no
 * cudaMalloc / cudaFree.  Meant for hosts that run under an arena or pool that forbids side
 * allocations, for latency-critical loops where an allocation could stall, and for embedders with
 * a fixed device budget.
 *   - limit: M * I * 2 bytes <= SFB200_NOALLOC_SCRATCH_BYTES, else SFB200_ERROR_SCRATCH_TOO_SMALL;
 *   - every GPU that loads the library holds the array until the process exits;
 *   - all calls on a device share the array: calls that overlap on the GPU race, serialise them;
 *   - the first call on a device resolves the array's device address: issue it before any stream
 *     capture begins;
 *   - "allocates nothing" covers this library's own calls; the CUDA runtime may still load a kernel's
 *     module at that kernel's first launch on a device (one more reason to call once at start-up).
 */
#define SFB200_NOALLOC_SCRATCH_BYTES (16u << 20)
SFB200_API int sfb200_ffn_forward_noalloc(const sfb200_ffn_weights* w, const void* x, int ldx, void* out,
                                          int ldo, int M, void* stream);
/* Status word of sfb200_ffn_forward_noalloc on the current device (no counterpart upstream): the
 * word lives in the library image like the scratch, so reading it allocates nothing either.
 * Synchronises the device, returns the word in *status_word (may be NULL) and clears it;
 * SFB200_ERROR_DEVICE when it was non-zero (a bounded wait inside that entry point's kernels ran
 * out: the output of that call is not valid).  0 when the entry point never ran on this device. */
SFB200_API int sfb200_noalloc_device_status(int* status_word);

/*
 * Persistent form of one compressed weight (host-only helpers, no GPU work): a 256-byte header
 * followed by the payload `values | pad to 256 | metadata`, i.e. the block sparseflow_sparse_gemm
 * takes as Bc.  The reference persists only dense copies and re-runs pruning and
 * to_sparse_semi_structured at every load (sparseflow/nn/sparseflow_linear.py:60-66); a host that
 * stores this blob skips both.  `layout_version` names the metadata tile layout: a reader that
 * gets SFB200_ERROR_NOT_SUPPORTED must re-compress from the dense weight.
 */
#define SFB200_BLOB_HEADER_BYTES 256
#define SFB200_LAYOUT_VERSION 1u
#define SFB200_BLOB_GATE_UP 1u /* rows are the 16-row interleaved gate|up order */
#define SFB200_BLOB_TIE_LOW 2u /* pruned with SFB200_TIE_LOW */
typedef struct {
  uint32_t layout_version;
  int32_t dtype, rows, K;
  uint32_t flags;
  uint64_t values_offset, values_bytes; /* offsets from the start of the blob */
  uint64_t meta_offset, meta_bytes;
  uint64_t total_bytes;
  uint64_t checksum; /* FNV-1a 64 of the payload, 0 = not recorded */
} sfb200_blob_info;
SFB200_API size_t sfb200_blob_bytes(int rows, int K); /* 0 for an unsupported shape */
SFB200_API uint64_t sfb200_blob_checksum(const void* payload_host, size_t bytes);
SFB200_API int sfb200_blob_write_header(void* header_host, int rows, int K, int dtype, unsigned flags,
                                        uint64_t checksum);
/* Validates magic, version, shape-derived sizes and that `available_bytes` holds the whole blob. */
SFB200_API int sfb200_blob_read_header(const void* header_host, size_t available_bytes,
                                       sfb200_blob_info* info);

/* Tuning hook: force the kernel variant / token tile on the current device.  0 = automatic;
 * 8 = decode kernel (M <= 32); 32/64/128/192/256 = single-CTA kernel with that token tile; 1256 =
 * CTA-pair kernel, 256-row x 256-token tiles; 1192/1208/1224/1240 = the same with that many tokens and
 * two accumulator sets; 5192/5208/5224/5240 = CTA-pair kernel, 512-row tiles with that many tokens and
 * 128-wide K stages (2192..2240: the same with 64-wide stages); 3032/3064/3128 and 4032/4064/4128 = split-K cluster kernel with 2 or 4
 * K slices and a 32/64/128-token tile.  No counterpart upstream. */
SFB200_API int sfb200_debug_force_token_tile(int bn);

/* Tuning hooks of the prefill kernel's tile order (process-wide; no counterpart upstream): l2_band_mb > 0 sets
 * the budget, in MB, of the band of the operand that is kept L2-resident (default 56); force_order picks that
 * operand: -1 automatic (the smaller of activations and compressed weight), 0 activations, 1 weights. */
SFB200_API int sfb200_debug_pair_tuning(int l2_band_mb, int force_order);

/* The variant the library picks on its own for Y[M, N] = X[M, K] . W^T (swiglu = 1: the fused gate|up GEMM,
 * N = 2 * I rows) on a GPU with num_sms SMs, in the numbering above; 0 for a non-positive size.  Host-only. */
SFB200_API int sfb200_debug_plan_gemm(int M, int N, int K, int swiglu, int num_sms);

/* Tuning hooks of sfb200_ffn_forward_host's copy/compute pipeline: tokens are processed in chunks
 * of `main_rows` while more than that remains, then the remainder is halved down to `tail_rows`
 * (small last chunks shorten what runs after the last host-to-device copy but run the GEMMs less
 * efficiently).  0 = default (1024 / 1024).  _chunk_plan is host-only and returns the number of chunks written to out8[8]. */
SFB200_API int sfb200_debug_host_pipeline(int main_rows, int tail_rows);
SFB200_API int sfb200_debug_host_chunk_plan(int M, int main_rows, int tail_rows, int* out8);

/* ------------------------------------------------------------------ 2. sf_* runtime API --- */
/* experiments/old_structure/runtime/api/sparseflow_api.h:8-28, exercised by tests/test_c_api.cpp. */

typedef struct {
  int32_t M, N, K;
  int32_t dtype;          /* 0 f16, 1 bf16, 2 f32   (runtime/benchmark/micro_bench.h:8)  */
  int32_t sparsity_type;  /* 0 dense, 1 2:4, 2 4:8  (micro_bench.h:9)                    */
  float sparsity_ratio;
  int32_t layout;         /* 0 row, 1 col           (micro_bench.h:10)                   */
} sf_matmul_desc;

typedef struct {
  int32_t sm_arch;
  int32_t num_sms;
  uint64_t shared_mem_kb;
} sf_gpu_info;

/* Kernel ids (micro_bench.h:20-25): 0 dense tensor-core, 1 hybrid, 2 sparse (tcgen05 prefill
 * kernel here), 3 sparse alternative (small-M kernel here). */
SFB200_API int32_t sf_select_kernel(const char* cache_path, const sf_matmul_desc* desc,
                                    const sf_gpu_info* gpu);
SFB200_API int32_t sf_cache_size(const char* cache_path);
SFB200_API void sf_cache_clear(const char* cache_path);

/*
 * C form of the dispatcher call that upstream only offers in C++,
 * KernelDispatcher::select_kernel(desc, gpu, A, B, C, stream)
 * (runtime/dispatch/kernel_dispatcher.cpp:42-188): d_weight = the DEVICE weight matrix [desc.M, desc.K]
 * (the 2:4 operand), d_x = activations [desc.N, desc.K], d_y = output [desc.N, desc.M]; any may be NULL.
 * With a weight, the "compression cached" eligibility rule is evaluated on its content (FNV-1a of the
 * first KiB + shape: runtime/cache/compressed_cache.cpp:9-29, kernel_dispatcher.cpp:67-80); when all
 * three are given, sparse and dense candidates are timed on them (and d_y is overwritten), otherwise on
 * synthetic buffers.  sf_select_kernel is this call with NULL matrices, as upstream
 * (api/sparseflow_api.cpp:44) -- through it alone a 2:4 shape is never eligible, upstream and here.
 */
SFB200_API int32_t sf_select_kernel_ex(const char* cache_path, const sf_matmul_desc* desc,
                                       const sf_gpu_info* gpu, const void* d_weight, const void* d_x,
                                       void* d_y);
/*
 * Content-keyed store of compressed weights (runtime/cache/compressed_cache.cpp:31-104; upstream fills
 * it inside its sparse launcher, kernels/sparse_cusparselt_24.cu:70-89).  Prunes + compresses the
 * DEVICE weight [desc.M, desc.K] into library-owned device buffers (layout of sfb200_sparse_gemm),
 * remembers them under (content hash, M, N, K, dtype, sparsity, device) and returns 1; a second call
 * with the same content returns the same buffers.  Returns 0 when the shape or dtype has no sparse
 * kernel, on a CUDA failure, or when the store would exceed its 1 GiB cap
 * (compressed_cache.cpp:42,70-74).  *values / *meta (may be NULL) receive the device pointers, owned by
 * the library until sf_compressed_cache_clear.  Synchronous.
 */
SFB200_API int32_t sf_compress_weight(const sf_matmul_desc* desc, const void* d_weight,
                                      const void** values, const void** meta);
SFB200_API int32_t sf_compressed_cache_count(void);  /* compressed_cache.cpp:94-97 */
SFB200_API uint64_t sf_compressed_cache_bytes(void); /* compressed_cache.cpp:89-92 */
SFB200_API void sf_compressed_cache_clear(void);     /* compressed_cache.cpp:83-87; frees the buffers */

/* Additions behind the same cache (no counterpart upstream; they make the dispatcher's
 * "compression cached" rule and failure quarantine reachable through the C ABI, which upstream
 * only reaches from C++: runtime/dispatch/kernel_dispatcher.cpp:67-98,165-174).
 * sf_note_compressed declares a shape's weight compressed without handing the matrix over. */
SFB200_API void sf_note_compressed(const char* cache_path, const sf_matmul_desc* desc);
SFB200_API void sf_record_sparse_failure(const char* cache_path, const sf_matmul_desc* desc,
                                         const sf_gpu_info* gpu);
SFB200_API int32_t sf_bucket_dimension(int32_t dim); /* kernel_dispatcher.cpp:16-28 */
/* Decision counters of the selector behind cache_path (upstream only prints "[Cache HIT]" etc. to
 * stdout, kernel_dispatcher.cpp:59,87,101): out[0..n) = calls, cache hits, misses, benchmark runs,
 * dense decisions, sparse decisions, sparse failures recorded, SPARSEFLOW_FORCE bypasses.  Returns
 * the number of counters written (at most 8). */
SFB200_API int32_t sf_get_counters(const char* cache_path, int64_t* out, int32_t n);
/* Environment: SPARSEFLOW_LOG=1 (decisions to stderr), SPARSEFLOW_CACHE_DB (database used for a NULL
 * cache_path instead of "kernel_cache.db"), SPARSEFLOW_FORCE=dense|sparse (every call returns 0, or 2
 * for shapes the sparse kernel supports, without lookup, measurement or persistence). */

/* ------------------------------------------------------------------ 3. C ABI v1 ----------- */
/* experiments/old_structure/include/sparseflow/c_api.h:38-200; src/runtime/context.cpp:78-300. */

#define SPARSEFLOW_ABI_VERSION_MAJOR 1
#define SPARSEFLOW_ABI_VERSION_MINOR 1 /* 1.1: adds SPARSEFLOW_DTYPE_BF16 */
#define SPARSEFLOW_ABI_VERSION_PATCH 0

typedef struct SparseFlowContext_* SparseFlowContext;
typedef struct SparseFlowKernel_* SparseFlowKernel;

typedef enum {
  SPARSEFLOW_SUCCESS = 0,
  SPARSEFLOW_ERROR_INVALID_ARGUMENT = 1,
  SPARSEFLOW_ERROR_OUT_OF_MEMORY = 2,
  SPARSEFLOW_ERROR_CUDA_ERROR = 3,
  SPARSEFLOW_ERROR_NOT_SUPPORTED = 4,
  SPARSEFLOW_ERROR_INVALID_HANDLE = 5,
  SPARSEFLOW_ERROR_COMPILATION_FAILED = 6,
  SPARSEFLOW_ERROR_ABI_MISMATCH = 7
} SparseFlowStatus;

typedef struct { int major; int minor; int patch; } SparseFlowVersion;

typedef enum {
  SPARSEFLOW_EPILOGUE_NONE = 0,
  SPARSEFLOW_EPILOGUE_RELU = 1,
  SPARSEFLOW_EPILOGUE_SILU = 2,
  SPARSEFLOW_EPILOGUE_GELU = 3,
  SPARSEFLOW_EPILOGUE_BIAS = 4,
  SPARSEFLOW_EPILOGUE_BIAS_RELU = 5,
  SPARSEFLOW_EPILOGUE_BIAS_SILU = 6
} SparseFlowEpilogue;

typedef struct {
  SparseFlowEpilogue kind;
  const void* params;  /* bias device pointer for the BIAS* kinds */
  size_t params_size;
} SparseFlowEpilogueConfig;

typedef struct {
  int tile_m, tile_n, tile_k; /* 0 = auto; tile_n in {32,64,128,192,256} picks the token tile */
  SparseFlowEpilogueConfig epilogue;
} SparseFlowKernelConfig;

typedef enum {
  SPARSEFLOW_DTYPE_FP16 = 0,
  SPARSEFLOW_DTYPE_FP32 = 1,
  SPARSEFLOW_DTYPE_INT8 = 2,
  SPARSEFLOW_DTYPE_BF16 = 3
} SparseFlowDataType;

typedef struct {
  double elapsed_ms;
  double tflops_effective;
  double tflops_real;
  double bandwidth_gb_s;
} SparseFlowBenchmarkResult;

SFB200_API const char* sparseflow_get_error_string(SparseFlowStatus status);     /* c_api.h:58 */
SFB200_API const char* sparseflow_get_last_error(void);                          /* c_api.h:61 */
SFB200_API SparseFlowVersion sparseflow_get_version(void);                       /* c_api.h:73 */
SFB200_API int sparseflow_is_abi_compatible(int major, int minor);               /* c_api.h:76 */
SFB200_API SparseFlowStatus sparseflow_create_context(SparseFlowContext* ctx, int device_id); /* :83 */
SFB200_API SparseFlowStatus sparseflow_destroy_context(SparseFlowContext ctx);   /* c_api.h:89 */
SFB200_API SparseFlowStatus sparseflow_get_device_info(SparseFlowContext ctx, int* compute_capability,
                                                       int* sm_count, size_t* total_memory); /* :94 */
SFB200_API SparseFlowStatus sparseflow_compile_kernel(SparseFlowContext ctx, SparseFlowKernel* kernel,
                                                      const SparseFlowKernelConfig* config); /* :131 */
SFB200_API SparseFlowStatus sparseflow_destroy_kernel(SparseFlowKernel kernel);  /* c_api.h:138 */
/*
 * C[M, N] = epilogue(A[M, K] . W^T), W = N x K weight compressed by sparseflow_compress_2_4.
 * `Bc` points at the compressed block: values (sfb200_values_bytes(N, K) bytes) followed, at the
 * next 256-byte boundary, by the metadata.  c_api.h:151-160 (a stub upstream, context.cpp:248).
 */
SFB200_API SparseFlowStatus sparseflow_sparse_gemm(SparseFlowKernel kernel, const void* A,
                                                   const void* Bc, void* C, int M, int N, int K,
                                                   SparseFlowDataType dtype, void* stream);
/* dense[M, N] -> compressed values + metadata; M rows, N = length of the pruned (K) axis.
 * c_api.h:163-169.  Prunes by magnitude first (idempotent on an already 2:4 tensor). */
SFB200_API SparseFlowStatus sparseflow_compress_2_4(SparseFlowContext ctx, const void* dense,
                                                    void* compressed, void* metadata, int M, int N,
                                                    SparseFlowDataType dtype);
/* Synchronous; is_valid is a HOST int.  c_api.h:172-177. */
SFB200_API SparseFlowStatus sparseflow_validate_2_4(const void* tensor, int M, int N,
                                                    SparseFlowDataType dtype, int* is_valid);
/* Times the sparse GEMM on library-owned synthetic buffers.  c_api.h:190-195. */
SFB200_API SparseFlowStatus sparseflow_benchmark_kernel(SparseFlowKernel kernel, int M, int N, int K,
                                                        int num_iterations,
                                                        SparseFlowBenchmarkResult* result);
/* Offset of the metadata inside the compressed block that sparseflow_sparse_gemm takes. */
SFB200_API size_t sparseflow_compressed_meta_offset(int N, int K);

#ifdef __cplusplus
}
#endif
#endif /* SPARSEFLOW_B200_H */
