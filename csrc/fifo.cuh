// Workspace layout and flow-control state of the Helix exchange.
//
// Every rank owns one workspace "row"; all rows are mapped at
// `workspace + rank * row_stride` in every process (or live in one tensor when a single
// process plays all ranks).  A row is laid out as
//
//   [ rings        : cp x maxC x 256 KiB ]  ring[sender][channel]: lines written by `sender`
//   [ sender info  : cp x maxC x 64 B    ]  sinfo[receiver][channel] = {head, tail}
//                                           head: lines this rank has sent on that ring (local)
//                                           tail: lines the receiver has consumed (stored remotely
//                                                 by the receiver, read only locally)
//   [ receiver info: cp x maxC x 64 B    ]  rinfo[sender][channel] = {tail}: lines consumed (local)
//   [ status       : 256 B               ]  StatusBlock, written when a bounded wait runs out
//   [ spare        : up to the row size  ]
//
// The row size keeps the reference's formula (csrc/helix_alltoall.cu:605-614):
// 512 KiB * cp * maxCh + 2 * 256 B * cp * maxCh with maxCh = max(SMs / (2 ceil(cp/8)), 1);
// this layout uses maxC = 2 * maxCh rings of half the size, one per SM on a 148-SM part.
//
// Rings are line rings: the line with absolute sequence q lives at slot q mod 2048 and
// carries flag q + 1, so a message may wrap around the end of the ring and consecutive
// launches simply continue where the previous one stopped (the reference instead burns a
// fresh 128 KiB FIFO entry per launch, csrc/helix_alltoall.cu:353-354,409-412).  As in
// the reference all polling is local and all remote traffic is posted stores
// (csrc/helix_alltoall.cu:386-388,446-449).
#pragma once

#include "helix_common.cuh"

namespace helix {

struct WorkspaceLayout {
  int cp;
  int max_channels;        // maxC
  int64_t ring_region;     // bytes
  int64_t sinfo_offset;    // byte offsets inside a row
  int64_t rinfo_offset;
  int64_t status_offset;
  int64_t row_bytes;       // size every caller must allocate per rank
};

HELIX_HD int ref_max_channel_count(int cp, int sm_count) {
  int blocks_per_channel = ceil_div(cp, 8) * 2;
  int c = sm_count / blocks_per_channel;
  return c > 1 ? c : 1;
}

HELIX_HD WorkspaceLayout make_layout(int cp, int sm_count) {
  WorkspaceLayout l;
  int max_ch_ref = ref_max_channel_count(cp, sm_count);
  l.cp = cp;
  l.max_channels = 2 * max_ch_ref;
  l.ring_region = (int64_t)kRingBytes * cp * l.max_channels;
  l.sinfo_offset = l.ring_region;
  l.rinfo_offset = l.sinfo_offset + (int64_t)kInfoSlotBytes * cp * l.max_channels;
  l.status_offset = l.rinfo_offset + (int64_t)kInfoSlotBytes * cp * l.max_channels;
  l.row_bytes = (int64_t)512 * 1024 * cp * max_ch_ref + (int64_t)2 * 256 * cp * max_ch_ref;
  return l;
}

// byte offset of ring[sender][channel] inside a row
HELIX_HD int64_t ring_offset(const WorkspaceLayout& l, int sender, int channel) {
  return ((int64_t)sender * l.max_channels + channel) * kRingBytes;
}
HELIX_HD int64_t sinfo_slot(const WorkspaceLayout& l, int receiver, int channel) {
  return l.sinfo_offset + ((int64_t)receiver * l.max_channels + channel) * kInfoSlotBytes;
}
HELIX_HD int64_t rinfo_slot(const WorkspaceLayout& l, int sender, int channel) {
  return l.rinfo_offset + ((int64_t)sender * l.max_channels + channel) * kInfoSlotBytes;
}

// Inside a sender-info slot: head at byte 0, tail at byte 32 (another 32-byte sector, so the
// remote store of tail never shares a sector with the locally written head).
constexpr int kSinfoHeadOff = 0;
constexpr int kSinfoTailOff = 32;
constexpr int kRinfoTailOff = 0;

// Flow-control rule: line q may be written once q - tail < kRingLines.
HELIX_HD bool ring_has_room(uint64_t q_last, uint64_t tail) {
  return q_last - tail < (uint64_t)kRingLines;
}

// entries of a call owned by channel c when `entries` are dealt round-robin over C channels
HELIX_HD int entries_of_channel(int entries, int channels, int c) {
  return c < entries ? (entries - c + channels - 1) / channels : 0;
}

}  // namespace helix
