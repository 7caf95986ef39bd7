// Shared constants, status codes and small device helpers of the Helix B200 kernels.
//
// Everything here compiles both as host C++ (g++) and as device code, so the
// protocol arithmetic can be unit-tested on a machine without a GPU.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define HELIX_HD __host__ __device__ __forceinline__
#define HELIX_D __device__ __forceinline__
#else
#define HELIX_HD inline
#define HELIX_D inline
#endif

namespace helix {

// ---- wire / ring geometry ---------------------------------------------------------------
constexpr int kLineBytes = 128;          // one NVLink-atomic store unit: 8 lanes x 16 B
constexpr int kLineWords = 16;           // u64 words per line
constexpr int kLineDataWords = 15;       // payload words per line; word 15 is the flag
constexpr int kLineDataBytes = 120;
constexpr int kChunkBytes = 16;          // what one lane stores / loads
constexpr int kChunksPerLine = 8;
constexpr int kRingBytes = 256 * 1024;   // one (sender, channel) ring in the receiver's row
constexpr int kRingLines = kRingBytes / kLineBytes;   // 2048, power of two
constexpr int kInfoSlotBytes = 64;       // one sender- or receiver-info slot
constexpr int kStatusBytes = 256;        // per-row status block
constexpr int kMaxEmulatedRanks = 8;     // ranks one launch can play in single-process mode
constexpr int kMaxCp = 32;
constexpr int kMaxRecvWarps = 8;

// ---- status codes written by a kernel whose bounded wait ran out -------------------------
enum Status : int {
  kOk = 0,
  kTimeoutRecv = 1,       // receiver: a line never showed its flag
  kTimeoutSendSpace = 2,  // sender: ring never drained (peer's receiver is stuck / absent)
  kTimeoutBarrier = 3,    // receiver-warps' software barrier
  kTimeoutGemmInput = 4,  // fused o_proj: activation tile never became ready
  kTimeoutMbarrier = 5,   // TMA / MMA mbarrier wait
  kBadArgument = 6,
};

// Layout of the status block (int64 words) at the start of the status region.
//  [0] code  [1] peer  [2] channel  [3] entry  [4] call counter  [5] last good call
struct StatusBlock {
  unsigned long long code;
  unsigned long long peer;
  unsigned long long channel;
  unsigned long long entry;
  unsigned long long calls;
  unsigned long long reserved[3];
};

HELIX_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }
HELIX_HD int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
HELIX_HD int64_t align_up64(int64_t a, int64_t b) { return ceil_div64(a, b) * b; }

}  // namespace helix
