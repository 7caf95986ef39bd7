// Peer-mapped workspace allocator built on the CUDA virtual-memory-management driver API.
//
// Every rank creates one physical allocation (its workspace row), exports a shareable
// handle, imports the handles of all peers and maps the rows at `base + rank * stride`
// inside one reserved virtual range, so the kernel reaches any row with plain pointer
// arithmetic.  The reference does the same from Python through cuda-python
// (helix_a2a/mnnvl.py:409-525); here it is C++, the driver entry points are resolved with
// cudaGetDriverEntryPoint (no link dependency on libcuda) and only the exchange of the
// handle bytes stays in Python (torch.distributed).
//
// Handle kinds: POSIX file descriptors (one box; duplicated into the importing process
// with pidfd_getfd, or passed over a Unix socket with SCM_RIGHTS) and fabric handles
// (64-byte blobs, multi-node NVLink).  A single process that drives several GPUs can map
// all of its rows itself (no handle exchange at all).
#pragma once

#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace helix {
namespace vmm {

enum HandleKind : int { kPosixFd = 0, kFabric = 1 };

struct Allocation;  // opaque

// Throws std::runtime_error with the driver's error name and a hint on failure.
Allocation* create(int cp_size, int cp_rank, int device, size_t row_bytes, HandleKind kind);

// The local row's shareable handle: for kPosixFd the decimal fd as text is NOT used; callers get
// the raw integer through export_fd(); for kFabric a 64-byte blob.
int export_fd(Allocation* a);
std::string export_fabric(Allocation* a);

// Map the local row at its slot.
void map_local(Allocation* a);
// Import a peer's handle and map its row.  `fd` must be valid in THIS process.
void map_peer_fd(Allocation* a, int peer_rank, int fd);
void map_peer_fabric(Allocation* a, int peer_rank, const std::string& blob);

// Duplicate file descriptor `fd` of process `pid` into this process (pidfd_open + pidfd_getfd).
int dup_fd_from_pid(int pid, int fd);
// SCM_RIGHTS transport over an abstract-namespace Unix socket.
void send_fd_unix(const std::string& name, int fd, int n_receivers, int timeout_ms);
int recv_fd_unix(const std::string& name, int timeout_ms);

// One process, several GPUs: rows of all devices mapped in one range, every device may access
// every row.  Returns the allocation that owns all rows.
Allocation* create_single_process(const std::vector<int>& devices, size_t row_bytes);

uint64_t base_address(const Allocation* a);
size_t row_stride(const Allocation* a);
size_t mapped_row_bytes(const Allocation* a);
int cp_size(const Allocation* a);
HandleKind kind(const Allocation* a);
bool fabric_supported(int device);

// Unmap everything, release the handles and free the reserved range.
void destroy(Allocation* a);

}  // namespace vmm
}  // namespace helix
