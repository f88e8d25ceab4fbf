// Device-side records shared by the plan kernel, the grouped expert GEMM and
// the host entry points.
#pragma once
#include <cuda.h>
#include <cstdint>

namespace mf {

constexpr int kMaxExperts = 256;   // routing limit (E <= 256, K <= 16), as in the reference router
constexpr int kMaxTopK = 16;
constexpr int kChunkTokens = 32;   // tokens per rank chunk of the stable pack

// Region of an expert's weights (the reference's indirection table: region 0
// is pinned host memory read over the link, 1 the HBM hot tier).
constexpr int kTierHost = 0;
constexpr int kTierHot = 1;

// One unit of grouped-GEMM work: a 128-row slice of one expert's weight (for
// w13: 64 gate rows and the matching 64 up rows) times up to n activation rows
// of that expert's packed segment.
struct GemmTile {
  int32_t w_row0;     // first output feature of the slice
  int32_t act_row0;   // first packed activation row
  int32_t rows;       // valid activation rows, 1..n
  int32_t n;          // MMA N = height of the activation box: 16/32/64/128/256
  int32_t z;          // slot of the expert inside its tier's weight tensor
  int32_t tier_phase; // kTierHost / kTierHot in bits 0..7, phase (0 = w13, 1 = w2) in bits 8..15
  int32_t expert;     // expert id (FP8 scale rows)
  int32_t block;      // row block id: w13 tiles count into done[block], w2 tiles wait on it
};
static_assert(sizeof(GemmTile) == 32, "GemmTile is 32 bytes");

// Queue state of one layer pass.  Written by the plan kernel.  Each tier has one
// queue holding all its w13 tiles followed by all its w2 tiles.
struct GemmQueues {
  int32_t n_tiles[2];      // [0 = link, 1 = hbm]
  int32_t head[2];         // next tile to hand out
  int32_t slots;           // link slots in use
  int32_t n_blocks;        // row blocks (entries of the done[] array in use)
  int32_t need;            // epilogue-warp arrivals that complete a row block's w13
  int32_t pad[9];
};
static_assert(sizeof(GemmQueues) == 64, "GemmQueues is 64 bytes");

constexpr int kActBoxes = 5;      // activation tensor maps with box heights 16, 32, 64, 128, 256

struct GemmPhaseParams {
  CUtensorMap w_map[2];            // [tier]: dims (K, rows, Z), box (64, 16, 1), 128-byte swizzle
  CUtensorMap w_map_big[2];        // the same tensors with box (64, 128, 1), for tiles without interleave
  CUtensorMap act_map[kActBoxes];  // dims (K, P), box (64, 16 << i), 128-byte swizzle
  const float* scale;              // FP8: fp32 [E][rows] per-output-channel scales, else null
  void* out;                       // w13: bf16 [P][ld_out]; w2: fp32 [P][ld_out]
  int32_t k_tiles;                 // K / 64
  int32_t up_offset;               // w13: first up row (= I)
  int32_t n_limit;                 // valid output features
  int32_t ld_out;
  int32_t scale_ld;                // row length of `scale`
  int32_t epi;
  int32_t packed[2];               // [tier] w13 only: rows stored as alternating 16-row gate / up groups
  int32_t w_fp8;                   // weights are e4m3 bytes (converted to bf16 in shared memory)
  int32_t pad[7];
};

struct GemmParams {
  GemmPhaseParams ph[2];           // [0 = w13, 1 = w2]
  const GemmTile* tiles[2];        // [0 = link, 1 = hbm]
  GemmQueues* q;
  int* done;                       // per row block: w13 epilogue arrivals
  int* status;                     // device error word (0 = ok)
  int32_t cap;                     // link credits: CTAs allowed to read host memory at once
  int32_t pad[3];
  unsigned long long* trace;       // debug: per-role event times of CTA 0 (u64 [4096]), or null
};

// Error bits in the device status word.
constexpr int kErrWaitTimeout = 1;   // a bounded mbarrier wait ran out
constexpr int kErrPlanOverflow = 2;  // more tiles than the plan buffers hold
constexpr int kErrBadArgs = 4;

}  // namespace mf
