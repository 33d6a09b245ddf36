// Internal launch interface between the C-ABI layer and the CUDA kernels.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sfb200 {

enum Err : int {
  kOk = 0,
  kErrInvalid = 1,
  kErrOutOfMemory = 2,
  kErrCuda = 3,
  kErrNotSupported = 4,
  kErrTensorMap = 8,
  kErrDevice = 9,     // a kernel reported a device-side failure through the status word
};

enum Fmt : int { kF16 = 0, kBF16 = 1 };
enum Epi : int { kEpiStore = 0, kEpiSwiGLU = 1 };
enum Act : int { kActNone = 0, kActRelu = 1, kActSilu = 2, kActGelu = 3 };
enum Tie : int { kTieHigh = 0, kTieLow = 1 };

// ---- prune + compress --------------------------------------------------------------------
struct PruneArgs {
  const void* dense;      // [rows, K] 16-bit, row pitch ld elements
  const void* dense2;     // optional second source (gate|up fusion), same shape, or null
  int rows;               // rows of ONE source
  int K;
  int ld;
  int fmt;
  int tie;
  int interleave;         // 0: out row r <- dense[r].  B>0 (needs dense2): blocks of B rows of
                          // `dense` followed by the matching B rows of `dense2`; out rows = 2*rows
  void* values;           // [out_rows, K/2]            or null
  void* meta;             // tiled metadata             or null
  void* ref_codes;        // [out_rows, K/4] uint8      or null
  void* pruned;           // [out_rows, K]              or null
};
int launch_prune_compress(const PruneArgs& a, cudaStream_t stream);
// one int result: 1 if every group of four has <= 2 non-zeros
int launch_validate_24(const void* w, int rows, int K, int ld, int* d_flag, cudaStream_t stream);
// rebuild pruned-dense [rows, K] from values + tiled metadata
int launch_decompress(const void* values, const void* meta, int rows, int K, void* dense, int ld,
                      cudaStream_t stream);

inline size_t values_bytes(int rows, int K) { return static_cast<size_t>(rows) * (K / 2) * 2; }
inline size_t meta_bytes(int rows, int K) {
  return static_cast<size_t>((rows + 127) / 128) * ((K + 127) / 128) * 2048;
}

// ---- sparse GEMM ---------------------------------------------------------------------------
struct SparseGemmArgs {
  const void* x;          // [m_tok, K], row pitch ldx
  const void* values;     // [n_out, K/2]
  const void* meta;       // tiled metadata of the n_out x K weight
  void* y;                // kEpiStore: [m_tok, n_out];  kEpiSwiGLU: [m_tok, n_out/2]; pitch ldy
  const void* bias;       // [n_out] or null (kEpiStore only)
  int* status;            // device status word
  int m_tok, n_out, K;
  int ldx, ldy;
  int fmt;
  int epi;
  int act;
  int num_sms;
  int force_bn;           // 0 = choose by token count
  int out_f32;            // 1: y is float [m_tok, ldy], results stored unrounded; 2: y is fp16 whatever the operand type,
                          // results clamped to the finite fp16 range (kEpiStore, CTA-pair kernel only)
  // Row-parallel GEMM of a tensor-parallel FFN with the reduce-scatter fused into the epilogue (CTA-pair kernel,
  // kEpiStore): token block o (tok_per_owner tokens, a multiple of 16) of this rank's partial output is stored to
  // peer_y[o] -- rank o's receive slot for this rank, [tok_per_owner, ldy], 16-bit or float per out_f32 -- instead of y.
  // peer_y: HOST array of tp device pointers (peer-mapped memory), or null.
  void* const* peer_y;
  int tp;
  int rank;               // this rank (peer_y set): its token tiles are visited starting at the next rank's block
  int tok_per_owner;
};
int launch_sparse_gemm(const SparseGemmArgs& a, cudaStream_t stream);
// CTA-pair (cta_group::2) kernel; launch_sparse_gemm goes straight to it from 4 * kPairMinTokens tokens and weighs it
// against the single-CTA tiles below that.  force_bn 1192..1256 (256-row tiles), 5192..5240 (512-row tiles, 128-wide
// K stages) or 2192..2240 (512-row tiles, 64-wide stages) picks a variant.
int launch_sparse_gemm_pair(const SparseGemmArgs& a, cudaStream_t stream);
constexpr int kPairMinTokens = 1024;
// Tuning hooks of the CTA-pair kernel's tile order: budget (MB) of the L2-resident operand's band (<= 0: keep),
// and which operand is resident (-1 automatic, 0 activations, 1 weights).  Process-wide.
void set_pair_tuning(int l2_band_mb, int force_order);
// Variant the CTA-pair launcher picks on its own (1192..1256 or 5192..5240; swiglu: the SiLU.mul epilogue) and,
// optionally, its estimated time in us.
int pick_pair_variant(int n_out, int m_tok, int K, int num_sms, int swiglu, double* cost_us = nullptr);
// The kernel variant launch_sparse_gemm runs for a shape when nothing is forced, in the numbering of
// SparseGemmArgs::force_bn: 8 decode kernel; 32..256 single-CTA kernel with that token tile; 1192..1256 / 5192..5240
// CTA-pair kernel; 3000 + tile / 4000 + tile split-K cluster kernel with 2 / 4 K slices.  Host-only.
int plan_sparse_gemm(int m_tok, int n_out, int K, int epi, int num_sms);
// The exchange step (reduction + all-gather) of the row-parallel GEMM in one launch per rank, cross-GPU ordering
// included.  mode 3: src = LOCAL receive slots [tp][slot_rows, cols] (slots_f32 = 0: 16-bit of the output type, 1: float, 2: fp16 whatever the output type) that the ranks' GEMM
// epilogues filled; the first `rows` rows of every slot are summed in fp32, bias added, rounded once and stored into
// every rank's output block (peer_dst[d], plain peer stores; or mc_dst, one multimem store).  mode 1 / 2: src = this
// rank's block inside the MULTICAST mapping of a symmetric buffer of 16-bit / float partial sums, summed inside
// NVSwitch; needs mc_dst.  mode 0: src = local 16-bit block, copied to every rank (all-gather).
// peer_flags: HOST array of tp device pointers, every rank's flag array of kSwitchFlagWords uint32 (zeroed once,
// symmetric memory); epoch: 1, 2, 3, ... one per launch on that flag array, the same on every rank.  Bounded waits; on
// a timeout the status word receives (2 << 8) | phase.
constexpr int kSwitchFlagWords = 2 * 148 * 8;
// Optional first phase of mode 3: the reduce-scatter as a copy, for a GEMM that wrote its partial sums locally.
struct ExchangePush {
  const void* src;              // local partial sums of this token chunk, owner blocks block_rows apart ([tp][block_rows, cols])
  void* const* peer_slots;      // HOST array: peer_slots[o] = where rank o keeps this rank's block (same type as the slots)
  int block_rows;
  int valid_rows[8];            // live rows of owner block o (0 .. block_rows)
  int light;                    // 1: 128-thread form that fits beside a GEMM CTA on an SM (for overlap on a side stream)
};
int launch_exchange(int mode, const void* src, void* mc_dst, void* const* peer_dst, int rows, int cols, int slot_rows,
                    int slots_f32, int fmt, const void* bias, void* const* peer_flags, int tp, int rank, unsigned epoch,
                    int* status, cudaStream_t stream, const ExchangePush* push = nullptr);

// Split-K variant of the single-CTA kernel: a cluster of `split` (2 or 4) CTAs shares one output tile,
// each streaming a slice of K; partial tiles are reduced through distributed shared memory.  Chosen by
// launch_sparse_gemm when splitk_factor() > 1 (too few row tiles to occupy the SMs).  kEpiStore only.
int launch_sparse_gemm_splitk(const SparseGemmArgs& a, int split, cudaStream_t stream);
int splitk_factor(int m_tok, int n_out, int K, int num_sms);
int splitk_token_tile(int m_tok);

// ---- small-M (decode) sparse GEMM ----------------------------------------------------------
// Supports M <= 32 tokens; chosen by launch_sparse_gemm for m_tok <= kSmallMMaxTokens (force_bn == 8 forces it).
int launch_sparse_gemm_small_m(const SparseGemmArgs& a, cudaStream_t stream);
constexpr int kSmallMMaxTokens = 4;   // from 5 tokens the tcgen05 kernel with a 32-token tile is faster (measured)

// ---- elementwise -----------------------------------------------------------------------------
// out[m, i] = silu(gu[m, i]) * gu[m, I + i]   (unfused variant, gate|up concatenated along columns)
int launch_silu_mul(const void* gate, const void* up, void* out, int rows, int cols, int ld_g,
                    int ld_u, int ld_o, int fmt, cudaStream_t stream);

}  // namespace sfb200
