#include "multicast_arena.hpp"

#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <mutex>

namespace geeps_b200 {

namespace {

// ---- driver entry points (the library links the static runtime only) ----
struct Drv {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  bool ok = false;
};

template <typename F>
bool load(F* fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  *fn = reinterpret_cast<F>(p);
  return true;
}

const Drv& drv() {
  static Drv d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = load(&d.MemCreate, "cuMemCreate") && load(&d.MemRelease, "cuMemRelease") &&
           load(&d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity") &&
           load(&d.MemAddressReserve, "cuMemAddressReserve") && load(&d.MemAddressFree, "cuMemAddressFree") &&
           load(&d.MemMap, "cuMemMap") && load(&d.MemUnmap, "cuMemUnmap") && load(&d.MemSetAccess, "cuMemSetAccess") &&
           load(&d.MemExportToShareableHandle, "cuMemExportToShareableHandle") &&
           load(&d.MemImportFromShareableHandle, "cuMemImportFromShareableHandle") &&
           load(&d.MulticastCreate, "cuMulticastCreate") && load(&d.MulticastAddDevice, "cuMulticastAddDevice") &&
           load(&d.MulticastBindMem, "cuMulticastBindMem") && load(&d.MulticastUnbind, "cuMulticastUnbind") &&
           load(&d.MulticastGetGranularity, "cuMulticastGetGranularity") && load(&d.DeviceGet, "cuDeviceGet") &&
           load(&d.DeviceGetAttribute, "cuDeviceGetAttribute");
  });
  return d;
}

std::string cu_err(const char* what, CUresult r) { return std::string(what) + " failed with CUresult " + std::to_string((int)r); }

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

bool map_rw(const Drv& d, CUdeviceptr* va, size_t bytes, CUmemGenericAllocationHandle h, int device, std::string* err,
            const char* what) {
  CUresult r = d.MemAddressReserve(va, bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMemAddressReserve", r); return false; }
  r = d.MemMap(*va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) { d.MemAddressFree(*va, bytes); *va = 0; *err = cu_err(what, r); return false; }
  CUmemAccessDesc a;
  memset(&a, 0, sizeof(a));
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = device;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.MemSetAccess(*va, bytes, &a, 1);
  if (r != CUDA_SUCCESS) { d.MemUnmap(*va, bytes); d.MemAddressFree(*va, bytes); *va = 0; *err = cu_err("cuMemSetAccess", r); return false; }
  return true;
}

// ---- file descriptors over Unix-domain sockets (abstract namespace: nothing is left in the file system) ----
struct FdMsg { int kind; int src; };     // kind 0: a rank's arena, 1: the multicast object

socklen_t uds_name(sockaddr_un* a, const std::string& tag, int rank) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  const std::string n = "geeps-mc-" + tag + "-" + std::to_string(rank);
  const size_t len = n.size() < sizeof(a->sun_path) - 2 ? n.size() : sizeof(a->sun_path) - 2;
  memcpy(a->sun_path + 1, n.data(), len);      // leading NUL byte: abstract socket
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + len);
}

bool send_fd(const std::string& tag, int to_rank, FdMsg m, int fd, std::string* err) {
  const int s = socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) { *err = "socket(AF_UNIX) failed"; return false; }
  sockaddr_un a;
  const socklen_t alen = uds_name(&a, tag, to_rank);
  int tries = 0;
  while (connect(s, reinterpret_cast<sockaddr*>(&a), alen) != 0) {
    if (++tries > 200) { close(s); *err = "cannot reach the handle listener of rank " + std::to_string(to_rank); return false; }
    usleep(20000);
  }
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec io{&m, sizeof(m)};
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  const bool ok = sendmsg(s, &msg, 0) == (ssize_t)sizeof(m);
  close(s);
  if (!ok) *err = "sendmsg(SCM_RIGHTS) failed";
  return ok;
}

bool recv_fd(int listen_fd, FdMsg* m, int* fd, int timeout_ms, std::string* err) {
  pollfd p{listen_fd, POLLIN, 0};
  if (poll(&p, 1, timeout_ms) <= 0) { *err = "timed out waiting for a peer's memory handle"; return false; }
  const int s = accept(listen_fd, nullptr, nullptr);
  if (s < 0) { *err = "accept on the handle listener failed"; return false; }
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec io{m, sizeof(*m)};
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  pollfd ps{s, POLLIN, 0};
  bool ok = poll(&ps, 1, timeout_ms) > 0 && recvmsg(s, &msg, 0) == (ssize_t)sizeof(*m);
  close(s);
  *fd = -1;
  if (ok) {
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    ok = c && c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS;
    if (ok) memcpy(fd, CMSG_DATA(c), sizeof(int));
  }
  if (!ok) *err = "no file descriptor in a peer's handle message";
  return ok;
}

}  // namespace

MulticastArena::~MulticastArena() { release(); }

bool MulticastArena::device_supported(int device) {
  const Drv& d = drv();
  if (!d.ok) return false;
  CUdevice dev;
  int v = 0;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
  return v != 0;
}

bool MulticastArena::allocate(size_t bytes, int device, std::string* err) {
  const Drv& d = drv();
  if (!d.ok) { *err = "CUDA driver entry points for virtual memory / multicast are not available"; return false; }
  device_ = device;
  const CUmemAllocationProp prop = alloc_prop(device);
  size_t gran = 0, mc_gran = 0;
  CUresult r = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMemGetAllocationGranularity", r); return false; }
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = 2;
  mp.size = gran;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  r = d.MulticastGetGranularity(&mc_gran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMulticastGetGranularity", r); return false; }
  if (mc_gran > gran) gran = mc_gran;
  bytes_ = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h = 0;
  r = d.MemCreate(&h, bytes_, &prop, 0);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMemCreate", r); return false; }
  mem_ = h;
  CUdeviceptr va = 0;
  if (!map_rw(d, &va, bytes_, h, device, err, "cuMemMap (own arena)")) { d.MemRelease(h); mem_ = 0; return false; }
  local_va_ = va;
  return true;
}

bool MulticastArena::listen(const std::string& tag, int rank, std::string* err) {
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM, 0);
  if (listen_fd_ < 0) { *err = "socket(AF_UNIX) failed"; return false; }
  sockaddr_un a;
  const socklen_t alen = uds_name(&a, tag, rank);
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&a), alen) != 0 || ::listen(listen_fd_, 32) != 0) {
    *err = std::string("cannot open the handle listener: ") + strerror(errno);
    close(listen_fd_);
    listen_fd_ = -1;
    return false;
  }
  return true;
}

bool MulticastArena::send_handles(const std::string& tag, int rank, int world, std::string* err) {
  const Drv& d = drv();
  int fd = -1;
  CUresult r = d.MemExportToShareableHandle(&fd, mem_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMemExportToShareableHandle (arena)", r); return false; }
  bool ok = true;
  for (int q = 0; q < world && ok; ++q)
    if (q != rank) ok = send_fd(tag, q, FdMsg{0, rank}, fd, err);
  close(fd);
  if (!ok) return false;
  if (rank == 0) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)world;
    mp.size = bytes_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle mc = 0;
    r = d.MulticastCreate(&mc, &mp);
    if (r != CUDA_SUCCESS) { *err = cu_err("cuMulticastCreate", r); return false; }
    mc_ = mc;
    int mfd = -1;
    r = d.MemExportToShareableHandle(&mfd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) { *err = cu_err("cuMemExportToShareableHandle (multicast object)", r); return false; }
    for (int q = 1; q < world && ok; ++q) ok = send_fd(tag, q, FdMsg{1, 0}, mfd, err);
    close(mfd);
  }
  return ok;
}

bool MulticastArena::receive_and_map(int rank, int world, std::string* err) {
  const Drv& d = drv();
  peer_mem_.assign((size_t)world, 0);
  peer_va_.assign((size_t)world, 0);
  peer_va_[(size_t)rank] = local_va_;
  const int expect = (world - 1) + (rank == 0 ? 0 : 1);
  for (int i = 0; i < expect; ++i) {
    FdMsg m{0, 0};
    int fd = -1;
    if (!recv_fd(listen_fd_, &m, &fd, 120000, err)) return false;
    CUmemGenericAllocationHandle h = 0;
    CUresult r = d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) { *err = cu_err("cuMemImportFromShareableHandle", r); return false; }
    if (m.kind == 1) { mc_ = h; continue; }
    if (m.src < 0 || m.src >= world || m.src == rank || peer_mem_[(size_t)m.src]) { d.MemRelease(h); *err = "unexpected handle message"; return false; }
    peer_mem_[(size_t)m.src] = h;
    CUdeviceptr va = 0;
    if (!map_rw(d, &va, bytes_, h, device_, err, "cuMemMap (peer arena)")) return false;
    peer_va_[(size_t)m.src] = va;
  }
  if (listen_fd_ >= 0) { close(listen_fd_); listen_fd_ = -1; }
  if (!mc_) { *err = "the multicast object never arrived"; return false; }
  CUdevice dev;
  CUresult r = d.DeviceGet(&dev, device_);
  if (r == CUDA_SUCCESS) r = d.MulticastAddDevice(mc_, dev);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMulticastAddDevice", r); return false; }
  mc_added_ = true;
  return true;
}

bool MulticastArena::bind_and_map(std::string* err) {
  const Drv& d = drv();
  CUresult r = d.MulticastBindMem(mc_, 0, mem_, 0, bytes_, 0);
  if (r != CUDA_SUCCESS) { *err = cu_err("cuMulticastBindMem", r); return false; }
  bound_ = true;
  CUdeviceptr va = 0;
  if (!map_rw(d, &va, bytes_, mc_, device_, err, "cuMemMap (multicast view)")) return false;
  mc_va_ = va;
  return true;
}

void MulticastArena::release() {
  const Drv& d = drv();
  if (!d.ok) return;
  if (listen_fd_ >= 0) { close(listen_fd_); listen_fd_ = -1; }
  if (mc_va_) { d.MemUnmap(mc_va_, bytes_); d.MemAddressFree(mc_va_, bytes_); mc_va_ = 0; }
  if (bound_) {
    CUdevice dev;
    if (d.DeviceGet(&dev, device_) == CUDA_SUCCESS) d.MulticastUnbind(mc_, dev, 0, bytes_);
    bound_ = false;
  }
  if (mc_) { d.MemRelease(mc_); mc_ = 0; }
  for (size_t r = 0; r < peer_va_.size(); ++r) {
    if (peer_mem_[r]) {
      if (peer_va_[r]) { d.MemUnmap(peer_va_[r], bytes_); d.MemAddressFree(peer_va_[r], bytes_); }
      d.MemRelease(peer_mem_[r]);
    }
  }
  peer_va_.clear();
  peer_mem_.clear();
  if (local_va_) { d.MemUnmap(local_va_, bytes_); d.MemAddressFree(local_va_, bytes_); local_va_ = 0; }
  if (mem_) { d.MemRelease(mem_); mem_ = 0; }
}

}  // namespace geeps_b200
