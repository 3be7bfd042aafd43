// Process-wide configuration read from environment variables.
//
// The reference parses its flags ad hoc in three places (src/env.cpp:11-33,
// src/ProcessGroupCCL.cpp:785-830,915-927, src/gpu/dpcpp_ccl.cpp:45-85,124-135, the last one
// with a getenv on every all-reduce). Here every knob is parsed once into one struct; `reparse()`
// exists for tests. Flag variables accept only integer strings, `1` means true, and a
// non-integer raises "Invalid value for environment variable: NAME" like the reference.
#pragma once
#include <cstdint>
#include <string>

namespace ccl {

struct Env {
  // names shared with intel/torch-ccl
  int verbose = 0;             // ONECCL_BINDINGS_FOR_PYTORCH_ENV_VERBOSE
  int wait_gdb = 0;            // ONECCL_BINDINGS_FOR_PYTORCH_ENV_WAIT_GDB
  bool llm_allreduce = false;  // TORCH_LLM_ALLREDUCE (implies same-stream)
  bool llm_allreduce_debug = false;  // TORCH_LLM_ALLREDUCE_DEBUG
  bool blocking_wait = false;  // CCL_BLOCKING_WAIT
  bool same_stream = false;    // CCL_SAME_STREAM
  bool disable_allreduce = false;  // TORCH_CCL_DISABLE_ALLREDUCE
  bool work_only = false;      // TORCH_CCL_WORK_ONLY
  bool sync_only = false;      // TORCH_CCL_SYNC_ONLY
  // knobs of this implementation
  std::string algo = "auto";   // CCL_ALGO = auto | oneshot | twoshot | nvls | nccl
  int64_t oneshot_max_bytes = -1;  // CCL_ONESHOT_MAX_BYTES (-1: tuner default)
  int nvls = 0;                // CCL_NVLS
  int64_t spin_timeout_ms = -1;  // CCL_SPIN_TIMEOUT_MS (-1: derived from the group timeout)
  bool debug_bounds = false;   // CCL_DEBUG_BOUNDS
  bool debug_checks = false;   // CCL_DEBUG_CHECKS: ranks compare {op, dtype, bytes} before every collective
  std::string tune_file;       // CCL_TUNE_FILE: per-world algorithm thresholds (see cuda/Tuner.h)
  std::string symm_mem = "ipc";  // CCL_SYMM_MEM = ipc | vmm: how CUDA arenas are shared
  int log_level = 0;           // CCL_LOG_LEVEL
  int64_t arena_mb = 256;      // CCL_ARENA_MB: one staging half per rank
  int64_t symm_heap_mb = 1024; // CCL_SYMM_HEAP_MB: symmetric heap for tensors allocated through the backend (created on first use)
  int64_t symm_min_bytes = -1; // CCL_SYMM_MIN_BYTES: smallest symmetric message that takes the zero-copy kernels (-1: built-in / tuning file)
  int64_t init_timeout_ms = -1; // CCL_INIT_TIMEOUT_MS: how long a rank waits for the others when the CPU communicator is built (-1: max(group timeout, 30 s))
  int64_t round_mb = -1;       // CCL_ROUND_MB: cap on the megabytes one staging round moves per rank (-1: built-in, 0: the arena half)
  int64_t nvls_min_bytes = -1; // CCL_NVLS_MIN_BYTES: smallest staged message that goes through the switch when CCL_NVLS=1 (-1: built-in / tuning file)
  int64_t shm_slot_mb = 4;     // CCL_SHM_SLOT_MB: CPU shared-memory slot per rank
  int max_blocks = -1;         // CCL_MAX_BLOCKS: CTAs of bandwidth-bound collectives (-1: 256 or the tuning file)
  int threads = -1;            // CCL_THREADS: threads per CTA of the collective kernels (-1: 512 or the tuning file)
  int local_rank = -1;         // LOCAL_RANK / MPI_LOCALRANKID / ...
  int local_world_size = -1;   // LOCAL_WORLD_SIZE / MPI_LOCALNRANKS / PALS_LOCAL_SIZE
  bool with_mpirun = false;

  static const Env& get();
  static void reparse();
};

// Parses a boolean flag variable with the reference's rules.
bool parse_env_flag(const char* name, bool default_value);
// Integer variable; returns `default_value` when unset, throws on non-integers.
int64_t parse_env_int(const char* name, int64_t default_value);

}  // namespace ccl
