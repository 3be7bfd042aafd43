// Stand-alone probes of the primitives the CUDA collectives are built on. No torch, no NCCL.
//
//   peer_probe ipc       two processes: the child maps the parent's buffer through a cudaIpc
//                        handle, reads it (map + remote read), then stores into it from a kernel
//                        and the parent checks that it sees the stores (remote store visibility)
//   peer_probe pingpong  two ranks bounce an epoch through a flag in each other's memory with
//                        st.release.sys / ld.acquire.sys and BOUNDED waits; prints the round trip.
//                        With >= 2 GPUs the ranks are two kernels on two GPUs of one process; with
//                        one GPU they are the two CTAs of one cooperative launch (kernels that wait
//                        for each other are never run as separate launches on one GPU)
//   peer_probe all       both
//
// Counterparts in intel/torch-ccl, all run by hand under `mpirun -n 2` and checked by eye:
// src/test/segfault/simple_test.cpp (map a peer buffer from an IPC handle and read it),
// src/test/writeremote/simple_test.cpp (write a peer buffer, peer checks),
// src/test/remotesync/simple_test.cpp (atomic flag written remotely, polled locally).
//
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o peer_probe peer_probe.cu
#include <cuda_runtime.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define CK(x)                                                                                   \
  do {                                                                                          \
    cudaError_t e_ = (x);                                                                       \
    if (e_ != cudaSuccess) {                                                                    \
      std::fprintf(stderr, "%s:%d: %s failed: %s\n", __FILE__, __LINE__, #x, cudaGetErrorString(e_)); \
      return 1;                                                                                 \
    }                                                                                           \
  } while (0)

namespace {

constexpr int kWords = 1 << 20;  // 4 MiB
constexpr long long kSpinBudgetCycles = 2000000000ll;  // about a second at 2 GHz

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *flag >= want or the cycle budget runs out; returns false on expiry.
__device__ bool bounded_wait(const uint32_t* flag, uint32_t want) {
  const long long t0 = clock64();
  while (ld_acquire_sys(flag) < want) {
    if (clock64() - t0 > kSpinBudgetCycles) return false;
  }
  return true;
}

__global__ void fill_kernel(uint32_t* p, int n, uint32_t seed) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = seed + (uint32_t)i;
}

// One side of the ping-pong. `mine` is the flag this rank polls (in its own memory), `theirs` the
// flag it writes (in the peer's memory). Rank 0 serves first.
__device__ void pingpong_side(int side, uint32_t* mine, uint32_t* theirs, int rounds, int* status) {
  for (int r = 1; r <= rounds; ++r) {
    if (side == 0) {
      st_release_sys(theirs, (uint32_t)r);
      if (!bounded_wait(mine, (uint32_t)r)) {
        *status = 100 + side;
        return;
      }
    } else {
      if (!bounded_wait(mine, (uint32_t)r)) {
        *status = 100 + side;
        return;
      }
      st_release_sys(theirs, (uint32_t)r);
    }
  }
}

// Two GPUs: one single-thread kernel per GPU.
__global__ void pingpong_kernel(int side, uint32_t* mine, uint32_t* theirs, int rounds, int* status) {
  pingpong_side(side, mine, theirs, rounds, status);
}

// One GPU: CTA b plays rank b; launched cooperatively so that both CTAs are resident.
__global__ void pingpong_coop_kernel(uint32_t* flags, int rounds, int* status) {
  if (threadIdx.x != 0) return;
  const int side = blockIdx.x;
  pingpong_side(side, flags + 32 * side, flags + 32 * (1 - side), rounds, status + side);
}

int ipc_child(int rd, int wr) {
  int ndev = 0;
  CK(cudaGetDeviceCount(&ndev));
  CK(cudaSetDevice(ndev > 1 ? 1 : 0));
  cudaIpcMemHandle_t h;
  if (read(rd, &h, sizeof(h)) != (ssize_t)sizeof(h)) return 1;
  void* remote = nullptr;
  CK(cudaIpcOpenMemHandle(&remote, h, cudaIpcMemLazyEnablePeerAccess));
  std::vector<uint32_t> host(kWords);
  CK(cudaMemcpy(host.data(), remote, kWords * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  int bad = 0;
  for (int i = 0; i < kWords; ++i) bad += host[i] != 0xA0000000u + (uint32_t)i;
  std::printf("[child ] mapped the parent's buffer and read %d words: %d mismatches\n", kWords, bad);
  fill_kernel<<<64, 256>>>(static_cast<uint32_t*>(remote), kWords, 0xB0000000u);  // remote stores
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  CK(cudaIpcCloseMemHandle(remote));
  const char ok = bad == 0 ? 'k' : 'x';
  if (write(wr, &ok, 1) != 1) return 1;
  return bad == 0 ? 0 : 1;
}

int run_ipc() {
  int to_child[2], to_parent[2];
  if (pipe(to_child) != 0 || pipe(to_parent) != 0) {
    std::perror("pipe");
    return 1;
  }
  const pid_t pid = fork();  // before any CUDA call: a CUDA context does not survive fork
  if (pid < 0) {
    std::perror("fork");
    return 1;
  }
  if (pid == 0) {
    const int rc = ipc_child(to_child[0], to_parent[1]);
    std::fflush(stdout);
    _exit(rc);  // never fall back into the parent's control flow
  }
  CK(cudaSetDevice(0));
  uint32_t* buf = nullptr;
  CK(cudaMalloc(&buf, kWords * sizeof(uint32_t)));
  fill_kernel<<<64, 256>>>(buf, kWords, 0xA0000000u);
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  CK(cudaIpcGetMemHandle(&h, buf));
  if (write(to_child[1], &h, sizeof(h)) != (ssize_t)sizeof(h)) return 1;
  char ok = 0;
  if (read(to_parent[0], &ok, 1) != 1) ok = 'x';
  int st = 0;
  waitpid(pid, &st, 0);
  std::vector<uint32_t> host(kWords);
  CK(cudaMemcpy(host.data(), buf, kWords * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  int bad = 0;
  for (int i = 0; i < kWords; ++i) bad += host[i] != 0xB0000000u + (uint32_t)i;
  std::printf("[parent] sees the child's remote stores: %d mismatches; child %s\n", bad,
              (ok == 'k' && WIFEXITED(st) && WEXITSTATUS(st) == 0) ? "ok" : "FAILED");
  CK(cudaFree(buf));
  return (bad == 0 && ok == 'k' && WIFEXITED(st) && WEXITSTATUS(st) == 0) ? 0 : 1;
}

int run_pingpong() {
  const int rounds = 2000;
  int ndev = 0;
  CK(cudaGetDeviceCount(&ndev));
  int* status = nullptr;  // host-mapped, so an expired wait is visible without touching the kernel
  CK(cudaHostAlloc(reinterpret_cast<void**>(&status), 2 * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
  status[0] = status[1] = 0;
  int can01 = 0, can10 = 0;
  if (ndev >= 2) {
    CK(cudaDeviceCanAccessPeer(&can01, 0, 1));
    CK(cudaDeviceCanAccessPeer(&can10, 1, 0));
  }
  float ms = 0.f;
  if (ndev >= 2 && can01 && can10) {
    uint32_t* flag[2];
    cudaStream_t s[2];
    cudaEvent_t e0, e1;
    for (int d = 0; d < 2; ++d) {
      CK(cudaSetDevice(d));
      cudaError_t pe = cudaDeviceEnablePeerAccess(1 - d, 0);
      if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) CK(pe);
      (void)cudaGetLastError();
      CK(cudaMalloc(&flag[d], 128));
      CK(cudaMemset(flag[d], 0, 128));
      CK(cudaStreamCreate(&s[d]));
    }
    for (int d = 0; d < 2; ++d) {
      CK(cudaSetDevice(d));
      CK(cudaDeviceSynchronize());
    }
    CK(cudaSetDevice(0));
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    int* dstatus = nullptr;
    CK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dstatus), status, 0));
    CK(cudaSetDevice(1));
    pingpong_kernel<<<1, 1, 0, s[1]>>>(1, flag[1], flag[0], rounds, dstatus + 1);
    CK(cudaGetLastError());
    CK(cudaSetDevice(0));
    CK(cudaEventRecord(e0, s[0]));
    pingpong_kernel<<<1, 1, 0, s[0]>>>(0, flag[0], flag[1], rounds, dstatus + 0);
    CK(cudaGetLastError());
    CK(cudaEventRecord(e1, s[0]));
    CK(cudaStreamSynchronize(s[0]));
    CK(cudaSetDevice(1));
    CK(cudaStreamSynchronize(s[1]));
    CK(cudaEventElapsedTime(&ms, e0, e1));
    std::printf("[pingpong] two GPUs over peer memory: ");
  } else {
    CK(cudaSetDevice(0));
    uint32_t* flags = nullptr;
    CK(cudaMalloc(&flags, 256));
    CK(cudaMemset(flags, 0, 256));
    int* dstatus = nullptr;
    CK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dstatus), status, 0));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    int r = rounds;
    void* args[] = {&flags, &r, &dstatus};
    CK(cudaEventRecord(e0));
    CK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(pingpong_coop_kernel), dim3(2), dim3(32), args, 0, nullptr));
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    CK(cudaEventElapsedTime(&ms, e0, e1));
    std::printf("[pingpong] one GPU, two CTAs of one cooperative launch: ");
  }
  const bool ok = status[0] == 0 && status[1] == 0;
  std::printf("%d round trips, %.2f us each, status %d/%d -> %s\n", rounds, ms * 1000.f / rounds, status[0], status[1],
              ok ? "ok" : "WAIT EXPIRED");
  return ok ? 0 : 1;
}

}  // namespace

int main(int argc, char** argv) {
  const char* mode = argc > 1 ? argv[1] : "all";
  int rc = 0;
  if (!std::strcmp(mode, "ipc") || !std::strcmp(mode, "all")) rc |= run_ipc();
  if (!std::strcmp(mode, "pingpong") || !std::strcmp(mode, "all")) rc |= run_pingpong();
  if (std::strcmp(mode, "ipc") && std::strcmp(mode, "pingpong") && std::strcmp(mode, "all")) {
    std::fprintf(stderr, "usage: %s [ipc|pingpong|all]\n", argv[0]);
    return 2;
  }
  std::printf("%s\n", rc == 0 ? "PASS" : "FAIL");
  return rc;
}
