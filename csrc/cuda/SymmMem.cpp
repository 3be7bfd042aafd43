#include "cuda/SymmMem.h"

#include <cuda.h>
#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace ccl {

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("ccl: ") + what + " failed: " + cudaGetErrorString(e));
}

[[noreturn]] void sys_fail(const std::string& what) {
  throw std::runtime_error("ccl: " + what + ": " + std::strerror(errno));
}

struct Fd {
  int fd = -1;
  Fd() = default;
  explicit Fd(int f) : fd(f) {}
  Fd(const Fd&) = delete;
  Fd& operator=(const Fd&) = delete;
  ~Fd() {
    if (fd >= 0) ::close(fd);
  }
};

// Abstract-namespace address (no file to clean up); returns the sockaddr length.
socklen_t abstract_addr(const std::string& name, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  if (name.size() + 1 > sizeof(addr->sun_path)) throw std::runtime_error("ccl: socket name too long");
  std::memcpy(addr->sun_path + 1, name.data(), name.size());
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

void send_fd(int sock, int rank, int fd) {
  int32_t payload = rank;
  iovec iov{&payload, sizeof(payload)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  ssize_t n;
  do {
    n = ::sendmsg(sock, &msg, MSG_NOSIGNAL);
  } while (n < 0 && errno == EINTR);
  if (n != static_cast<ssize_t>(sizeof(payload))) sys_fail("sendmsg(SCM_RIGHTS)");
}

int recv_fd(int sock, int* src_rank) {
  int32_t payload = -1;
  iovec iov{&payload, sizeof(payload)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t n;
  do {
    n = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  } while (n < 0 && errno == EINTR);
  if (n != static_cast<ssize_t>(sizeof(payload))) sys_fail("recvmsg(SCM_RIGHTS)");
  int fd = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
  }
  if (fd < 0) throw std::runtime_error("ccl: peer message carried no file descriptor");
  *src_rank = payload;
  return fd;
}

bool wait_readable(int fd, std::chrono::steady_clock::time_point deadline) {
  for (;;) {
    const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now());
    if (left.count() <= 0) return false;
    pollfd p{fd, POLLIN, 0};
    const int r = ::poll(&p, 1, static_cast<int>(std::min<int64_t>(left.count(), 1000)));
    if (r > 0) return true;
    if (r < 0 && errno != EINTR) sys_fail("poll");
  }
}

}  // namespace

void barrier_kv(KvStore& kv, const std::string& key, int world, uint64_t timeout_ms) {
  if (!kv.add) return;
  kv.add(key, 1);
  const auto t0 = std::chrono::steady_clock::now();
  while (kv.add(key, 0) < world) {
    if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms))
      throw std::runtime_error("ccl: timeout in bootstrap barrier '" + key + "'");
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
}

std::vector<int> exchange_fds(KvStore& kv, const std::string& prefix, int rank, int world, int my_fd,
                              uint64_t timeout_ms) {
  std::vector<int> out(world, -1);
  out[rank] = ::fcntl(my_fd, F_DUPFD_CLOEXEC, 0);
  if (out[rank] < 0) sys_fail("dup");
  if (world == 1) return out;
  static std::atomic<uint64_t> serial{0};
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  try {
    Fd listener(::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0));
    if (listener.fd < 0) sys_fail("socket(AF_UNIX)");
    const std::string name = "ccl-fdx-" + std::to_string(::getpid()) + "-" + std::to_string(serial.fetch_add(1)) + "-" +
                             std::to_string(rank);
    sockaddr_un addr;
    socklen_t len = abstract_addr(name, &addr);
    if (::bind(listener.fd, reinterpret_cast<sockaddr*>(&addr), len) != 0) sys_fail("bind(" + name + ")");
    if (::listen(listener.fd, world + 4) != 0) sys_fail("listen");
    kv.set(prefix + "/fdsock/" + std::to_string(rank), std::vector<uint8_t>(name.begin(), name.end()));

    // send to every peer: connect() and the small sendmsg() complete against the peer's backlog
    // and socket buffer, so this loop never waits for the peer's accept()
    for (int i = 1; i < world; ++i) {
      const int p = (rank + i) % world;
      const std::vector<uint8_t> pn = kv.get(prefix + "/fdsock/" + std::to_string(p));
      sockaddr_un pa;
      socklen_t pl = abstract_addr(std::string(pn.begin(), pn.end()), &pa);
      Fd s(::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0));
      if (s.fd < 0) sys_fail("socket(AF_UNIX)");
      for (;;) {
        if (::connect(s.fd, reinterpret_cast<sockaddr*>(&pa), pl) == 0) break;
        if (errno != EINTR && errno != EAGAIN && errno != ECONNREFUSED) sys_fail("connect(fd exchange)");
        if (std::chrono::steady_clock::now() > deadline) throw std::runtime_error("ccl: timeout connecting to peer for fd exchange");
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      send_fd(s.fd, rank, my_fd);
    }
    for (int got = 0; got < world - 1; ++got) {
      if (!wait_readable(listener.fd, deadline)) throw std::runtime_error("ccl: timeout waiting for a peer's file descriptor");
      Fd c(::accept4(listener.fd, nullptr, nullptr, SOCK_CLOEXEC));
      if (c.fd < 0) sys_fail("accept");
      if (!wait_readable(c.fd, deadline)) throw std::runtime_error("ccl: timeout waiting for a peer's file descriptor");
      int src = -1;
      const int fd = recv_fd(c.fd, &src);
      if (src < 0 || src >= world || src == rank || out[src] >= 0) {
        ::close(fd);
        throw std::runtime_error("ccl: unexpected sender in fd exchange");
      }
      out[src] = fd;
    }
    // keep the listener alive until every peer has connected
    barrier_kv(kv, prefix + "/fdsock/done", world, timeout_ms);
  } catch (...) {
    for (int f : out)
      if (f >= 0) ::close(f);
    throw;
  }
  return out;
}

SymmKind parse_symm_kind(const std::string& s) {
  if (s.empty() || s == "ipc") return SymmKind::kIpc;
  if (s == "vmm") return SymmKind::kVmm;
  throw std::runtime_error("ccl: CCL_SYMM_MEM must be 'ipc' or 'vmm', got '" + s + "'");
}

// ---------------------------------------------------------------------------------------------
// Driver entry points, resolved through the runtime so that the library does not link libcuda.

namespace {

struct Driver {
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExport = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImport = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGranularity = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;

  template <typename F>
  static void load(const char* name, F* fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    check(cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q), name);
    if (q != cudaDriverEntryPointSuccess || !p) throw std::runtime_error(std::string("ccl: driver entry point not found: ") + name);
    *fn = reinterpret_cast<F>(p);
  }

  Driver() {
    load("cuMemCreate", &MemCreate);
    load("cuMemRelease", &MemRelease);
    load("cuMemAddressReserve", &MemAddressReserve);
    load("cuMemAddressFree", &MemAddressFree);
    load("cuMemMap", &MemMap);
    load("cuMemUnmap", &MemUnmap);
    load("cuMemSetAccess", &MemSetAccess);
    load("cuMemExportToShareableHandle", &MemExport);
    load("cuMemImportFromShareableHandle", &MemImport);
    load("cuMemGetAllocationGranularity", &MemGranularity);
    load("cuGetErrorString", &GetErrorString);
    load("cuDeviceGet", &DeviceGet);
    load("cuDeviceGetAttribute", &DeviceGetAttribute);
    load("cuMulticastCreate", &MulticastCreate);
    load("cuMulticastAddDevice", &MulticastAddDevice);
    load("cuMulticastBindMem", &MulticastBindMem);
    load("cuMulticastUnbind", &MulticastUnbind);
    load("cuMulticastGetGranularity", &MulticastGetGranularity);
  }

  void ok(CUresult r, const char* what) const {
    if (r == CUDA_SUCCESS) return;
    const char* msg = nullptr;
    GetErrorString(r, &msg);
    throw std::runtime_error(std::string("ccl: ") + what + " failed: " + (msg ? msg : "unknown driver error"));
  }
};

const Driver& driver() {
  static Driver d;
  return d;
}

}  // namespace

bool SymmMem::multicast_supported(int device) {
  const Driver& d = driver();
  CUdevice dev;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  int ok = 0;
  if (d.DeviceGetAttribute(&ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
  return ok != 0;
}

SymmMem::SymmMem(SymmKind kind, int rank, int world, int device, size_t bytes, KvStore& kv, const std::string& prefix,
                 bool multicast)
    : kind_(kind), rank_(rank), world_(world), device_(device), bytes_(bytes), mapped_(bytes) {
  bases_.assign(world_, nullptr);
  check(cudaSetDevice(device_), "cudaSetDevice");
  check(cudaFree(nullptr), "context creation");
  if (multicast && kind_ != SymmKind::kVmm) throw std::runtime_error("ccl: multicast needs CCL_SYMM_MEM=vmm");
  if (kind_ == SymmKind::kIpc)
    init_ipc(kv, prefix);
  else
    init_vmm(kv, prefix, multicast && world_ > 1 && multicast_supported(device_));  // an object needs >= 2 devices
  // nobody may write into a buffer before its owner has zeroed it and everyone has mapped it
  if (world_ > 1) barrier_kv(kv, prefix + "/ready", world_, 120000);
}

void SymmMem::init_ipc(KvStore& kv, const std::string& prefix) {
  void* base = nullptr;
  check(cudaMalloc(&base, bytes_), "cudaMalloc(symmetric memory)");
  bases_[rank_] = base;
  check(cudaMemset(base, 0, bytes_), "cudaMemset(symmetric memory)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (world_ == 1) return;
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, base), "cudaIpcGetMemHandle");
  std::vector<uint8_t> blob(sizeof(h) + sizeof(int));
  std::memcpy(blob.data(), &h, sizeof(h));
  std::memcpy(blob.data() + sizeof(h), &device_, sizeof(int));
  kv.set(prefix + "/ipc/" + std::to_string(rank_), blob);
  for (int p = 0; p < world_; ++p) {
    if (p == rank_) continue;
    std::vector<uint8_t> pb = kv.get(prefix + "/ipc/" + std::to_string(p));
    if (pb.size() != blob.size()) throw std::runtime_error("ccl: malformed IPC handle from peer");
    cudaIpcMemHandle_t ph;
    int pdev = 0;
    std::memcpy(&ph, pb.data(), sizeof(ph));
    std::memcpy(&pdev, pb.data() + sizeof(ph), sizeof(int));
    int can = 0;
    if (pdev != device_) check(cudaDeviceCanAccessPeer(&can, device_, pdev), "cudaDeviceCanAccessPeer");
    if (!can && pdev != device_)
      throw std::runtime_error("ccl: GPU " + std::to_string(device_) + " cannot access peer GPU " + std::to_string(pdev));
    void* pp = nullptr;
    check(cudaIpcOpenMemHandle(&pp, ph, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    bases_[p] = pp;
  }
}

void SymmMem::init_vmm(KvStore& kv, const std::string& prefix, bool multicast) {
  const Driver& d = driver();
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  d.ok(d.MemGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (gran == 0) gran = 2u << 20;
  if (multicast) {
    // the bound range must also be a multiple of the multicast granularity
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)world_;
    mp.size = bytes_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    d.ok(d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    if (mg > gran) gran = (mg + gran - 1) / gran * gran;
  }
  mapped_ = (bytes_ + gran - 1) / gran * gran;
  handles_.assign(world_, 0);

  CUmemGenericAllocationHandle own = 0;
  d.ok(d.MemCreate(&own, mapped_, &prop, 0), "cuMemCreate");
  handles_[rank_] = own;

  CUmemAccessDesc access;
  std::memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;

  auto map = [&](CUmemGenericAllocationHandle h) -> void* {
    CUdeviceptr va = 0;
    d.ok(d.MemAddressReserve(&va, mapped_, gran, 0, 0), "cuMemAddressReserve");
    d.ok(d.MemMap(va, mapped_, 0, h, 0), "cuMemMap");
    d.ok(d.MemSetAccess(va, mapped_, &access, 1), "cuMemSetAccess");
    return reinterpret_cast<void*>(va);
  };
  bases_[rank_] = map(own);
  check(cudaMemset(bases_[rank_], 0, mapped_), "cudaMemset(symmetric memory)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (world_ == 1) {
    if (multicast) init_multicast(kv, prefix, gran);
    return;
  }

  int fd = -1;
  d.ok(d.MemExport(&fd, own, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  std::vector<int> fds;
  try {
    fds = exchange_fds(kv, prefix + "/vmm", rank_, world_, fd, 120000);
  } catch (...) {
    ::close(fd);
    throw;
  }
  ::close(fd);
  try {
    for (int p = 0; p < world_; ++p) {
      if (p == rank_) continue;
      CUmemGenericAllocationHandle h = 0;
      d.ok(d.MemImport(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[p])), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
           "cuMemImportFromShareableHandle");
      handles_[p] = h;
      bases_[p] = map(h);
    }
  } catch (...) {
    for (int f : fds) ::close(f);
    throw;
  }
  for (int f : fds) ::close(f);  // the imported handles keep the memory alive
  if (multicast) init_multicast(kv, prefix, gran);
}

// One multicast object for the communicator: rank 0 creates it and hands its descriptor to the
// others; every rank adds its device, then (once all devices are in) binds its own allocation and
// maps the object. A store through the mapping lands in every rank's allocation, a
// multimem.ld_reduce through it returns the sum over all of them.
void SymmMem::release_multicast() {
  const Driver& d = driver();
  if (mc_base_) {
    d.MemUnmap(reinterpret_cast<CUdeviceptr>(mc_base_), mapped_);
    d.MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_base_), mapped_);
    mc_base_ = nullptr;
  }
  if (mc_handle_) {
    CUdevice dev;
    if (mc_bound_ && d.DeviceGet(&dev, device_) == CUDA_SUCCESS) d.MulticastUnbind(mc_handle_, dev, 0, mapped_);
    mc_bound_ = false;
    d.MemRelease(mc_handle_);
    mc_handle_ = 0;
  }
}

void SymmMem::init_multicast(KvStore& kv, const std::string& prefix, size_t gran) {
  // a process must never go away with its memory still bound to the object: undo on any failure
  try {
    init_multicast_impl(kv, prefix, gran);
  } catch (...) {
    release_multicast();
    throw;
  }
}

void SymmMem::init_multicast_impl(KvStore& kv, const std::string& prefix, size_t gran) {
  const Driver& d = driver();
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = (unsigned)world_;
  mp.size = mapped_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mc = 0;
  if (rank_ == 0) {
    d.ok(d.MulticastCreate(&mc, &mp), "cuMulticastCreate");
    mc_handle_ = mc;
  }
  if (world_ > 1) {
    // all-gather of descriptors; only rank 0's matters, the others pass their own allocation's
    int fd = -1;
    d.ok(d.MemExport(&fd, rank_ == 0 ? mc : (CUmemGenericAllocationHandle)handles_[rank_], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
         "cuMemExportToShareableHandle(multicast)");
    std::vector<int> fds;
    try {
      fds = exchange_fds(kv, prefix + "/mc", rank_, world_, fd, 120000);
    } catch (...) {
      ::close(fd);
      throw;
    }
    ::close(fd);
    CUresult r = CUDA_SUCCESS;
    if (rank_ != 0)
      r = d.MemImport(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[0])), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    for (int f : fds) ::close(f);
    d.ok(r, "cuMemImportFromShareableHandle(multicast)");
  }
  mc_handle_ = mc;
  CUdevice dev;
  d.ok(d.DeviceGet(&dev, device_), "cuDeviceGet");
  d.ok(d.MulticastAddDevice(mc, dev), "cuMulticastAddDevice");
  // memory may be bound only after every device has been added
  if (world_ > 1) barrier_kv(kv, prefix + "/mc/added", world_, 120000);
  d.ok(d.MulticastBindMem(mc, 0, (CUmemGenericAllocationHandle)handles_[rank_], 0, mapped_, 0), "cuMulticastBindMem");
  mc_bound_ = true;
  if (world_ > 1) barrier_kv(kv, prefix + "/mc/bound", world_, 120000);
  CUmemAccessDesc access;
  std::memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUdeviceptr va = 0;
  d.ok(d.MemAddressReserve(&va, mapped_, gran, 0, 0), "cuMemAddressReserve(multicast)");
  d.ok(d.MemMap(va, mapped_, 0, mc, 0), "cuMemMap(multicast)");
  d.ok(d.MemSetAccess(va, mapped_, &access, 1), "cuMemSetAccess(multicast)");
  mc_base_ = reinterpret_cast<void*>(va);
}

SymmMem::~SymmMem() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  if (kind_ == SymmKind::kIpc) {
    for (int p = 0; p < world_; ++p)
      if (p != rank_ && bases_[p]) cudaIpcCloseMemHandle(bases_[p]);
    if (bases_[rank_]) cudaFree(bases_[rank_]);
    return;
  }
  const Driver& d = driver();
  // multicast first: unmap the view, unbind this device's memory, drop the object
  release_multicast();
  for (int p = 0; p < world_; ++p) {
    if (bases_[p]) {
      d.MemUnmap(reinterpret_cast<CUdeviceptr>(bases_[p]), mapped_);
      d.MemAddressFree(reinterpret_cast<CUdeviceptr>(bases_[p]), mapped_);
    }
    if (p < static_cast<int>(handles_.size()) && handles_[p]) d.MemRelease(handles_[p]);
  }
}

}  // namespace ccl
