// Data layouts shared by the host side of the fabric and its persistent kernel.
//
// The wire formats a caller sees — the 64-byte tile descriptor, the 8-int stage
// row, the successor list, the worker->lane map, the host mirror — are those of
// the reference fabric (csrc/fabric/types.h:13-111), because its Python program
// builder (monoserve/fabric/program.py) packs them and its engine reads them.
// Everything else (rings, lane state, worker layout) is this library's own.
#pragma once
#include <cstdint>

namespace mf {
namespace fab {

constexpr int kMaxLanes = 4;
constexpr int kMaxWorkers = 256;
constexpr uint32_t kRingCap = 1u << 14;   // activated stages per ring
constexpr uint32_t kNoLane = 0xffu;

// Tile kinds.  0..4 are the fabric's own; model tiles start at 32
// (csrc/fabric/types.h:19-26, csrc/fabric/model_types.h:8-24).
enum TileKind : uint16_t {
  kTileNop = 0,
  kTileSpin = 1,          // a[0] ns, a[1] trace base, i0 trace index, i1 lane tag
  kTileRead = 2,          // a[0] source, a[1] bytes, a[2] sink, a[3] trace base, i0 trace index
  kTileProbe = 3,         // a[0] chain base, i0 loads, a[1] result, i1 result index
  kTileZeroRuntime = 4,   // re-arm stages [i0, i1) except i2
  kTileGemm = 32,
  kTileAttnPrefill = 33,    // an attention work item (prefill and decode items share one code path)
  kTileAttnDecode = 34,
  kTileAttnMerge = 35,      // merge of the key ranges of a split item
  kTileRmsNorm = 36,
  kTileQkRope = 37,
  kTileRouter = 38,
  kTileExpand = 39,
  kTilePermute = 40,
  kTileAddNorm = 41,
  kTileEmbed = 42,
  kTileSample = 43,
  kTileAttnPlan = 44,
  kTileGemmAsym = 45,       // a K range of a 128-row weight slice against ALL i2 rows of its expert, in blocks of bm rows
  kTileAsymReduce = 46,     // rows [i0, i0 + i1): h = silu(gate) * up from fp32 partial sums, which are zeroed
  kTileCombine = 47,        // not in the reference: un-permute + weighted combine in pick order (+ RMSNorm)
  kTileRouterLogits = 48,   // not in the reference: router projection with a defined summation order
  kTileFetch = 49,          // not in the reference: a[0] source, a[1] destination, i0 bytes; host memory -> HBM staging
  kTileNormLogits = 50,     // not in the reference: for rows [i0, i0 + i1) the norm tile (a[0] NormArgs, kind a[3] = 36
                            // or 41 with slabs) and then the router projection of those rows against experts
                            // [i2, i2 + i3) (a[1] LogitsArgs): the norm stage of a small batch folded into the
                            // projection's tiles (every expert-range tile of a row group writes the same norm)
};
constexpr int kFabChunk = 16;   // rows per router / permute tile = rank chunk of the stable pack

enum StageFlags : uint32_t {
  kStageLink = 1u << 0,   // tiles read host memory: taken only under a link slot
  kStageReset = 1u << 1,  // completion ends one iteration of the program
  kStageMark = 1u << 2,   // completion is reported to the host (mark value)
  kStageSkip = 1u << 3,   // out of this iteration
};

struct alignas(64) TileDesc {
  uint16_t kind;
  uint8_t lane;
  uint8_t flags;
  uint32_t stage;
  uint32_t i0, i1, i2, i3;
  uint64_t a[5];
};
static_assert(sizeof(TileDesc) == 64, "TileDesc is 64 bytes");

struct alignas(32) StageStatic {
  uint32_t first, count, succ_first, succ_count, deps_init, flags, mark, pad;
};
static_assert(sizeof(StageStatic) == 32, "StageStatic is 32 bytes");

// tag_next = iteration tag << 32 | index of the next tile to hand out.
struct alignas(16) StageRuntime {
  unsigned long long tag_next;
  unsigned int done;
  unsigned int deps;
};
static_assert(sizeof(StageRuntime) == 16, "StageRuntime is 16 bytes");

struct alignas(64) ProgramDesc {
  TileDesc* tiles;
  StageStatic* stages;
  StageRuntime* runtime;
  uint32_t* succ;
  uint32_t n_tiles, n_stages, first_stage, reset_stage;
  uint32_t iterations;   // 0: repeat until a newer program replaces it
  uint32_t gen;          // unique per upload
};

// The plan the host publishes as an epoch; double-buffered on the device.
struct alignas(128) Snapshot {
  unsigned long long epoch;
  uint32_t n_workers, n_lanes;
  uint32_t cap[kMaxLanes];        // link slots per lane
  uint32_t order[kMaxLanes];      // lanes in borrowing order
  uint32_t prog_gen[kMaxLanes];
  uint32_t form[kMaxLanes];       // kernel form of host-resident experts: 16/32/64/128, 0 = weight-stationary
  ProgramDesc* prog[kMaxLanes];
  uint8_t map[kMaxWorkers];       // worker -> lane, kNoLane = none
};

// Written by the device into pinned host memory.
struct alignas(64) LaneMirror {
  unsigned long long iterations, gen, running, mark, mark_ns, iter_ns;
  unsigned long long pad[2];
};
struct alignas(64) HostMirror {
  LaneMirror lane[kMaxLanes];
  unsigned long long worker_epoch[kMaxWorkers];
  unsigned long long worker_epoch_ns[kMaxWorkers];
  unsigned long long error;       // first device error (kFabErr* bits), 0 = none
  unsigned long long pad[7];
};

// Device error bits (HostMirror::error, DeviceState::error).
constexpr unsigned long long kFabErrRingWait = 1;     // a ring publication waited longer than its budget
constexpr unsigned long long kFabErrWorklist = 2;     // more simultaneously completed stages than the worklist holds
constexpr unsigned long long kFabErrDeadline = 4;     // the kernel reached its run-time limit and left
constexpr unsigned long long kFabErrBadTile = 8;      // a tile kind this build does not execute
constexpr unsigned long long kFabErrTileWait = 16;    // a bounded wait inside a tile ran out
constexpr unsigned long long kFabErrDynOverflow = 32; // the expander needs more tiles than the dynamic region holds

struct alignas(128) Ring {
  unsigned long long head;
  unsigned long long pad0[15];
  unsigned long long reserve;
  unsigned long long pad1[15];
  unsigned long long tail;
  unsigned long long pad2[15];
  unsigned int ids[kRingCap];
};

struct alignas(128) LaneState {
  Ring ring[2];                   // [0] ungated stages, [1] link stages
  unsigned int slots;             // link slots held
  unsigned int inflight;          // link tiles executing now
  unsigned int inflight_max;
  unsigned int running;           // 1 while the lane has an active program
  unsigned int tag;               // iteration tag of the current activation wave
  unsigned int iter_in_prog;
  unsigned int gen;
  unsigned int pad;
  unsigned long long prog;        // const ProgramDesc* of the active program
};

struct alignas(128) DeviceState {
  LaneState lane[kMaxLanes];
  Snapshot snap[2];
  unsigned long long published;   // current epoch; the host writes it last
  unsigned int shutdown;
  unsigned int idle_cap;          // longest idle back-off, ns
  unsigned int trace_cap, trace_n;
  unsigned long long trace_ptr;   // u64 [trace_cap][2] stage events
  unsigned long long max_run_ns;  // the kernel leaves on its own after this long (0 = no limit)
  unsigned long long error;
  HostMirror* mirror;
  unsigned long long worker_tile[kMaxWorkers];
  unsigned long long worker_tile_ns[kMaxWorkers];
  // Written when a worker leaves after a bounded wait ran out: where its roles were waiting.
  // Four words per worker: [0] TMA producer, [1] MMA, [2] first exec warp, each
  // record << 48 | q phases << 40 | phases[0] << 32 | phases[1] << 24 | tile << 8 | site
  // (sites in attention_core.cuh; 13 = the producer's drain), [3] records finished by the
  // exec warps | by the MMA warp << 32.
  unsigned long long worker_wait[kMaxWorkers][4];
};

// Per-tile trace record of the test tiles (csrc/fabric/core_tiles.cuh:10-17).
struct alignas(32) TraceRec {
  unsigned long long start_ns, end_ns;
  unsigned int worker, sm, count, lane;
};

}  // namespace fab
}  // namespace mf
