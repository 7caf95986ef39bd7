// CUDA VMM workspace allocator (see vmm_workspace.h).
#include "vmm_workspace.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/syscall.h>
#include <sys/un.h>
#include <unistd.h>

#include <mutex>
#include <sstream>
#include <stdexcept>

namespace helix {
namespace vmm {
namespace {

// ---- driver entry points ---------------------------------------------------------------------
struct Driver {
  CUresult (*GetErrorName)(CUresult, const char**) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
};

template <class F>
void resolve(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || p == nullptr || q != cudaDriverEntryPointSuccess)
    throw std::runtime_error(std::string("helix vmm: CUDA driver entry point not available: ") + name);
  fn = reinterpret_cast<F>(p);
}

Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    resolve(d.GetErrorName, "cuGetErrorName");
    resolve(d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    resolve(d.MemAddressReserve, "cuMemAddressReserve");
    resolve(d.MemAddressFree, "cuMemAddressFree");
    resolve(d.MemCreate, "cuMemCreate");
    resolve(d.MemRelease, "cuMemRelease");
    resolve(d.MemMap, "cuMemMap");
    resolve(d.MemUnmap, "cuMemUnmap");
    resolve(d.MemSetAccess, "cuMemSetAccess");
    resolve(d.MemExportToShareableHandle, "cuMemExportToShareableHandle");
    resolve(d.MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    resolve(d.DeviceGetAttribute, "cuDeviceGetAttribute");
  });
  return d;
}

void check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* name = nullptr;
  drv().GetErrorName(r, &name);
  std::ostringstream os;
  os << "helix vmm: " << what << " failed: " << (name ? name : "unknown") << " (" << (int)r << ")";
  if (r == CUDA_ERROR_NOT_PERMITTED)
    os << " - for fabric handles check that the IMEX daemon runs and its channel device is visible";
  if (r == CUDA_ERROR_NOT_SUPPORTED) os << " - this handle type is not supported on this GPU / driver";
  throw std::runtime_error(os.str());
}

void check_rt(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("helix vmm: ") + what + ": " + cudaGetErrorString(e));
}

CUmemAllocationProp make_prop(int device, HandleKind kind) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = kind == kFabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

constexpr size_t kSlotAlign = size_t(1) << 29;  // rows start on 512 MiB boundaries of the reserved range

}  // namespace

struct Allocation {
  int cp = 0, rank = 0;
  HandleKind kind = kPosixFd;
  std::vector<int> devices;                          // device of each row we created (1 entry normally)
  CUdeviceptr base = 0;
  size_t stride = 0, row = 0, reserved = 0;
  std::vector<CUmemGenericAllocationHandle> handles;  // per rank (0 = not mapped)
  std::vector<bool> mapped;
  int export_fd = -1;
};

static void set_access(Allocation* a, int slot, const std::vector<int>& devs) {
  std::vector<CUmemAccessDesc> acc(devs.size());
  for (size_t i = 0; i < devs.size(); ++i) {
    memset(&acc[i], 0, sizeof(CUmemAccessDesc));
    acc[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc[i].location.id = devs[i];
    acc[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  }
  check(drv().MemSetAccess(a->base + a->stride * slot, a->row, acc.data(), acc.size()), "cuMemSetAccess");
}

static Allocation* reserve(int cp, size_t row_bytes, const CUmemAllocationProp& prop) {
  Allocation* a = new Allocation();
  size_t gran = 0;
  check(drv().MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
        "cuMemGetAllocationGranularity");
  a->cp = cp;
  a->row = (row_bytes + gran - 1) / gran * gran;
  a->stride = (a->row + kSlotAlign - 1) / kSlotAlign * kSlotAlign;
  a->reserved = a->stride * cp;
  a->handles.assign(cp, 0);
  a->mapped.assign(cp, false);
  try {
    check(drv().MemAddressReserve(&a->base, a->reserved, kSlotAlign, 0, 0), "cuMemAddressReserve");
  } catch (...) {
    delete a;
    throw;
  }
  return a;
}

Allocation* create(int cp_size, int cp_rank, int device, size_t row_bytes, HandleKind kind) {
  if (cp_size < 1 || cp_rank < 0 || cp_rank >= cp_size) throw std::runtime_error("helix vmm: bad cp_size / cp_rank");
  check_rt(cudaSetDevice(device), "cudaSetDevice");
  check_rt(cudaFree(nullptr), "context creation");
  CUmemAllocationProp prop = make_prop(device, kind);
  Allocation* a = reserve(cp_size, row_bytes, prop);
  a->rank = cp_rank;
  a->kind = kind;
  a->devices = {device};
  try {
    check(drv().MemCreate(&a->handles[cp_rank], a->row, &prop, 0), "cuMemCreate");
  } catch (...) {
    destroy(a);
    throw;
  }
  return a;
}

int export_fd(Allocation* a) {
  if (a->kind != kPosixFd) throw std::runtime_error("helix vmm: allocation does not use POSIX fd handles");
  if (a->export_fd < 0) {
    int fd = -1;
    check(drv().MemExportToShareableHandle(&fd, a->handles[a->rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
          "cuMemExportToShareableHandle(fd)");
    a->export_fd = fd;
  }
  return a->export_fd;
}

std::string export_fabric(Allocation* a) {
  if (a->kind != kFabric) throw std::runtime_error("helix vmm: allocation does not use fabric handles");
  CUmemFabricHandle h;
  check(drv().MemExportToShareableHandle(&h, a->handles[a->rank], CU_MEM_HANDLE_TYPE_FABRIC, 0),
        "cuMemExportToShareableHandle(fabric)");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void map_local(Allocation* a) {
  int r = a->rank;
  if (a->mapped[r]) return;
  check(drv().MemMap(a->base + a->stride * r, a->row, 0, a->handles[r], 0), "cuMemMap(local)");
  a->mapped[r] = true;
  set_access(a, r, a->devices);
}

static void map_imported(Allocation* a, int peer, CUmemGenericAllocationHandle h) {
  a->handles[peer] = h;
  check(drv().MemMap(a->base + a->stride * peer, a->row, 0, h, 0), "cuMemMap(peer)");
  a->mapped[peer] = true;
  set_access(a, peer, a->devices);
}

void map_peer_fd(Allocation* a, int peer_rank, int fd) {
  if (peer_rank < 0 || peer_rank >= a->cp || peer_rank == a->rank || a->mapped[peer_rank])
    throw std::runtime_error("helix vmm: bad peer rank in map_peer_fd");
  CUmemGenericAllocationHandle h = 0;
  check(drv().MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle(fd)");
  map_imported(a, peer_rank, h);
}

void map_peer_fabric(Allocation* a, int peer_rank, const std::string& blob) {
  if (peer_rank < 0 || peer_rank >= a->cp || peer_rank == a->rank || a->mapped[peer_rank])
    throw std::runtime_error("helix vmm: bad peer rank in map_peer_fabric");
  if (blob.size() != sizeof(CUmemFabricHandle)) throw std::runtime_error("helix vmm: fabric handle must be 64 bytes");
  CUmemFabricHandle fh;
  memcpy(&fh, blob.data(), sizeof(fh));
  CUmemGenericAllocationHandle h = 0;
  check(drv().MemImportFromShareableHandle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC), "cuMemImportFromShareableHandle(fabric)");
  map_imported(a, peer_rank, h);
}

int dup_fd_from_pid(int pid, int fd) {
#ifndef SYS_pidfd_open
#define SYS_pidfd_open 434
#endif
#ifndef SYS_pidfd_getfd
#define SYS_pidfd_getfd 438
#endif
  long pidfd = syscall(SYS_pidfd_open, pid, 0);
  if (pidfd < 0) {
    int e = errno;
    throw std::runtime_error("helix vmm: pidfd_open(" + std::to_string(pid) + ") failed: " + strerror(e) +
                             " - ranks must share a PID namespace (one box, --ipc=host)");
  }
  long got = syscall(SYS_pidfd_getfd, (int)pidfd, fd, 0);
  int e = errno;
  close((int)pidfd);
  if (got < 0) {
    std::string msg = "helix vmm: pidfd_getfd failed: " + std::string(strerror(e));
    if (e == EPERM) msg += " - needs CAP_SYS_PTRACE; set HELIX_A2A_HANDLE_TRANSPORT=scm to pass descriptors over a socket";
    throw std::runtime_error(msg);
  }
  return (int)got;
}

// ---- SCM_RIGHTS transport -----------------------------------------------------------------------
static sockaddr_un abstract_addr(const std::string& name, socklen_t* len) {
  sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  size_t n = std::min(name.size(), sizeof(addr.sun_path) - 2);
  memcpy(addr.sun_path + 1, name.data(), n);  // leading NUL: abstract namespace, nothing on disk
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
  return addr;
}

void send_fd_unix(const std::string& name, int fd, int n_receivers, int timeout_ms) {
  int srv = socket(AF_UNIX, SOCK_STREAM, 0);
  if (srv < 0) throw std::runtime_error("helix vmm: socket() failed");
  socklen_t len;
  sockaddr_un addr = abstract_addr(name, &len);
  if (bind(srv, (sockaddr*)&addr, len) != 0 || listen(srv, n_receivers + 1) != 0) {
    int e = errno;
    close(srv);
    throw std::runtime_error(std::string("helix vmm: bind/listen failed: ") + strerror(e));
  }
  for (int i = 0; i < n_receivers; ++i) {
    pollfd pfd{srv, POLLIN, 0};
    if (poll(&pfd, 1, timeout_ms) <= 0) {
      close(srv);
      throw std::runtime_error("helix vmm: timed out waiting for a peer to fetch the descriptor");
    }
    int c = accept(srv, nullptr, nullptr);
    if (c < 0) continue;
    char byte = 'h';
    iovec iov{&byte, 1};
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(cm), &fd, sizeof(int));
    sendmsg(c, &msg, 0);
    close(c);
  }
  close(srv);
}

int recv_fd_unix(const std::string& name, int timeout_ms) {
  socklen_t len;
  sockaddr_un addr = abstract_addr(name, &len);
  int waited = 0;
  while (true) {
    int s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) throw std::runtime_error("helix vmm: socket() failed");
    if (connect(s, (sockaddr*)&addr, len) == 0) {
      char byte;
      iovec iov{&byte, 1};
      char ctrl[CMSG_SPACE(sizeof(int))];
      msghdr msg{};
      msg.msg_iov = &iov;
      msg.msg_iovlen = 1;
      msg.msg_control = ctrl;
      msg.msg_controllen = sizeof(ctrl);
      pollfd pfd{s, POLLIN, 0};
      int fd = -1;
      if (poll(&pfd, 1, timeout_ms) > 0 && recvmsg(s, &msg, 0) > 0) {
        cmsghdr* cm = CMSG_FIRSTHDR(&msg);
        if (cm && cm->cmsg_type == SCM_RIGHTS) memcpy(&fd, CMSG_DATA(cm), sizeof(int));
      }
      close(s);
      if (fd < 0) throw std::runtime_error("helix vmm: peer did not send a descriptor");
      return fd;
    }
    close(s);
    if (waited >= timeout_ms) throw std::runtime_error("helix vmm: timed out connecting to " + name);
    usleep(2000);
    waited += 2;
  }
}

Allocation* create_single_process(const std::vector<int>& devices, size_t row_bytes) {
  if (devices.empty()) throw std::runtime_error("helix vmm: no devices");
  int cur = 0;
  check_rt(cudaGetDevice(&cur), "cudaGetDevice");
  for (int d : devices) {
    check_rt(cudaSetDevice(d), "cudaSetDevice");
    check_rt(cudaFree(nullptr), "context creation");
  }
  CUmemAllocationProp prop0 = make_prop(devices[0], kPosixFd);
  Allocation* a = reserve((int)devices.size(), row_bytes, prop0);
  a->devices = devices;
  a->rank = -1;
  try {
    for (size_t i = 0; i < devices.size(); ++i) {
      CUmemAllocationProp prop = make_prop(devices[i], kPosixFd);
      check(drv().MemCreate(&a->handles[i], a->row, &prop, 0), "cuMemCreate");
      check(drv().MemMap(a->base + a->stride * i, a->row, 0, a->handles[i], 0), "cuMemMap");
      a->mapped[i] = true;
      set_access(a, (int)i, devices);
    }
  } catch (...) {
    destroy(a);
    cudaSetDevice(cur);
    throw;
  }
  cudaSetDevice(cur);
  return a;
}

uint64_t base_address(const Allocation* a) { return (uint64_t)a->base; }
size_t row_stride(const Allocation* a) { return a->stride; }
size_t mapped_row_bytes(const Allocation* a) { return a->row; }
int cp_size(const Allocation* a) { return a->cp; }
HandleKind kind(const Allocation* a) { return a->kind; }

bool fabric_supported(int device) {
  int v = 0;
  if (drv().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, device) != CUDA_SUCCESS) return false;
  return v != 0;
}

void destroy(Allocation* a) {
  if (!a) return;
  // Kernels of THIS process that still use the rows must be over before the mappings go away (a handle that is
  // dropped while an exchange is in flight would otherwise unmap memory under it).  Peers that may still be
  // storing into our row are the caller's business: barrier over the group before closing a workspace.
  cudaDeviceSynchronize();
  for (int i = 0; i < a->cp; ++i) {
    if (a->mapped[i]) drv().MemUnmap(a->base + a->stride * i, a->row);
    if (a->handles[i]) drv().MemRelease(a->handles[i]);
  }
  if (a->base) drv().MemAddressFree(a->base, a->reserved);
  if (a->export_fd >= 0) close(a->export_fd);
  delete a;
}

}  // namespace vmm
}  // namespace helix
