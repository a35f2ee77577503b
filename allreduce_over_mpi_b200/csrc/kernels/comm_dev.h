// Structures shared by the communicator runtime (host) and the collective kernels.
#pragma once
#include <stdint.h>

#include "../api/ft_types.h"

namespace ftk {

constexpr int kMaxLanes = 512;     // CTAs of one collective kernel
constexpr int kMaxStages = 128;    // ring over 64 ranks has 126

struct Status {          // lives in pinned host memory, read by the host after a sync
  int code;              // ft_status; first failure wins
  int index;             // rendezvous index inside the call
  int peer;
  int lane;
  unsigned int calls;    // bumped by lane 0 of every collective kernel (progress marker)
};

typedef unsigned long long flag_t;
constexpr flag_t kCallStride = 256;  // rendezvous numbers reserved per call (> kMaxStages + 2)


// Per-rank view of the world: where every rank's symmetric heap and flag array are
// mapped in THIS process, plus local bookkeeping.  Passed by value to every kernel.
struct CommDev {
  unsigned char* heap[FT_MAX_RANKS];   // heap[r] = base of rank r's symmetric heap (peer mapping)
  unsigned long long* flags[FT_MAX_RANKS];  // flags[r] = rank r's flag array [kMaxLanes][FT_MAX_RANKS]
  unsigned char* mc_heap;              // multicast mapping of the heaps (NVLS), or null
  unsigned long long* call_count;      // local: number of collective calls so far (read by every CTA)
  unsigned int* arrived;               // local: CTAs of the running kernel that have read call_count
  Status* status;                      // pinned host memory
  int rank, world;
  unsigned long long timeout_ns;
  uint64_t heap_bytes;                 // bytes of every rank's heap mapping (what the FT_BOUNDS build checks against)
};

// One pull of the plan, device form.
struct DevPull {
  uint16_t block;
  uint8_t nsrc;
  uint8_t reduce;
  uint8_t src[FT_MAX_FANIN];
  uint16_t slot;          // tagged-word protocol: receive slot of src[0] on this rank (src[k] lands in slot + k)
};
// The same edge seen from its source, for the tagged-word (push) form of a plan: in this stage the rank
// sends its current copy of `block` into receive slot `slot` of rank `dst`.
struct DevPush {
  uint16_t block;
  uint16_t slot;
  uint8_t dst;
};
struct DevStage {
  uint32_t pull_begin, pull_end;
  uint32_t push_begin, push_end;   // range in the rank's DevPush table
  uint64_t sync_mask;     // ranks met before this stage
  uint32_t last_rs;       // 1 when this is the final reduce-scatter stage (scale applies here)
  uint32_t is_ag;
};
struct DevPlan {
  uint32_t nstages, npulls;
  uint32_t npushes, nslots;        // tagged-word form: pushes of this rank, receive slots it needs
  uint64_t end_sync_mask;
  DevStage stages[kMaxStages];
  // DevPull pulls[npulls] follow
};

// Arguments of one staged all-reduce launch.
struct StagedArgs {
  const DevPlan* plan;
  const DevPull* pulls;
  uint64_t work_off;          // byte offset of the work buffer inside every rank's heap
  uint64_t alt_stride;        // staging mode: odd calls use work_off + alt_stride (double buffer); else 0
  const void* user_in;        // not null: copied into the work buffer first (lane-sliced)
  void* user_out;             // not null: every finished block is also written here
  uint64_t count;             // elements
  uint64_t block_elems;       // elements per block (block bytes are a multiple of 16)
  uint32_t elem_size;
  uint32_t stage_begin, stage_end;   // [begin, end) — the full plan unless emulating
  uint32_t do_sync;           // 0: no rendezvous at all (single-GPU emulation, one stage per launch)
  uint32_t end_sync;          // closing rendezvous: 0 none, 1 the plan's set after the last stage, 2 every rank (a phase run alone)
  uint32_t user_vec_ok;       // user_in / user_out are 16-byte aligned
  float scale;                // applied when a block's reduction completes (float types)
};

struct OneShotArgs {
  uint64_t slot_off;          // byte offset of staging slot 0 in every heap (slot 1 follows it)
  uint64_t emu_call;          // call number to assume when the rendezvous phase is off (emulation)
  const void* user_in;
  void* user_out;
  uint64_t count;
  uint32_t elem_size;
  uint32_t phase_mask;        // bit0 copy-in, bit1 rendezvous, bit2 reduce (all three normally)
  uint32_t user_vec_ok;
  float scale;
};

// Low-latency push all-reduce: data travels as 8-byte words {32 data bits, 32-bit tag}.
constexpr uint64_t kLLMaxBytes = 256 << 10;             // largest message (payload bytes)
constexpr uint64_t kLLSrcStride = 2 * kLLMaxBytes;      // wire bytes one source rank may deposit per parity
struct LLArgs {
  uint64_t ll_off;            // byte offset of the receive area in every heap: [2 parities][world][kLLSrcStride]
  const void* user_in;
  void* user_out;
  uint64_t count;
  uint32_t elem_size;
  uint32_t phase_mask;        // bit0 send, bit1 receive+reduce (both normally; split only for emulation)
  uint32_t user_vec_ok;
  uint32_t use_call_counter;  // 0: take the call number from emu_call (emulation)
  uint64_t emu_call;
  float scale;
};

// A plan run with the tagged-word protocol (small messages): every edge of a stage is a push of 8-byte words
// {32 data bits, 32-bit tag} into a receive slot of the destination, so a tree level costs one one-way NVLink
// trip and no rendezvous.  One thread owns 16-byte item i of every block from the first stage to the last.
struct LLTreeArgs {
  const DevPlan* plan;
  const DevPull* pulls;
  const DevPush* pushes;
  uint64_t ll_off;            // receive area in every heap: [2 parities][world * kLLSrcStride]
  const void* user_in;
  void* user_out;
  uint64_t count;
  uint64_t block_elems;
  uint32_t elem_size;
  uint32_t stage_begin, stage_end;
  uint32_t phase_mask;        // bit0 push, bit1 receive (both normally; split only for single-GPU emulation)
  uint32_t user_vec_ok;
  uint32_t use_call_counter;
  uint64_t emu_call;
  float scale;
  uint32_t table_bytes;       // > 0: the kernel keeps the plan's tables in this much dynamic shared memory ...
  uint32_t table_counts[3];   // ... holding this many stages, pulls and pushes
};

struct NvlsArgs {
  uint64_t work_off;
  uint64_t count;
  uint64_t block_elems;
  uint64_t stripe_bytes;      // NVLS all-reduce only: 0 = rank r owns block r; else stripes of this size dealt round-robin
  uint32_t elem_size;
  float scale;
};

// Launch shape of the NVLS kernels (tuning knobs of the communicator).
// Measured on 8 B200 (64 MiB - 1 GiB) once every lane's slice starts on a 1 KiB boundary: the bus bandwidth sits on a
// plateau (683 / 806 / 839 GB/s at 64 MiB / 256 MiB / 1 GiB) for anything between 16 and 64 CTAs of 128-512 threads with
// 2-4 vectors in flight; 512 threads x 4 vectors on all 148 SMs fall off it (585 / 767 / 744).  The small launch also
// leaves three quarters of the SMs to whatever else is running (a backward pass).
struct NvlsConfig {
  int threads = 256;          // per CTA
  int unroll = 4;             // 16-byte vectors in flight per thread
  int weak = 0;               // 1: multimem.*.weak instead of .relaxed.sys
};

}  // namespace ftk
