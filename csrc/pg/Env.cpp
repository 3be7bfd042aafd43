#include "pg/Env.h"

#include <c10/util/Exception.h>

#include <cstdlib>
#include <mutex>

namespace ccl {

int64_t parse_env_int(const char* name, int64_t default_value) {
  const char* s = std::getenv(name);
  if (s == nullptr) return default_value;
  try {
    size_t pos = 0;
    const long long v = std::stoll(s, &pos);
    return static_cast<int64_t>(v);
  } catch (std::exception&) {
    TORCH_CHECK(false, "Invalid value for environment variable: " + std::string(name));
  }
}

bool parse_env_flag(const char* name, bool default_value) {
  const char* s = std::getenv(name);
  if (s == nullptr) return default_value;
  return parse_env_int(name, 0) == 1;
}

namespace {

std::mutex g_mu;
Env g_env;
bool g_parsed = false;

std::string env_str(const char* name, const std::string& def) {
  const char* s = std::getenv(name);
  return s ? std::string(s) : def;
}

Env parse() {
  Env e;
  e.verbose = (int)parse_env_int("ONECCL_BINDINGS_FOR_PYTORCH_ENV_VERBOSE", 0);
  e.wait_gdb = (int)parse_env_int("ONECCL_BINDINGS_FOR_PYTORCH_ENV_WAIT_GDB", 0);
  e.llm_allreduce = parse_env_flag("TORCH_LLM_ALLREDUCE", false);
  e.llm_allreduce_debug = parse_env_flag("TORCH_LLM_ALLREDUCE_DEBUG", false);
  e.blocking_wait = parse_env_flag("CCL_BLOCKING_WAIT", false);
  e.same_stream = parse_env_flag("CCL_SAME_STREAM", false) || e.llm_allreduce;
  e.disable_allreduce = parse_env_flag("TORCH_CCL_DISABLE_ALLREDUCE", false);
  e.work_only = parse_env_flag("TORCH_CCL_WORK_ONLY", false);
  e.sync_only = parse_env_flag("TORCH_CCL_SYNC_ONLY", false);
  e.algo = env_str("CCL_ALGO", "auto");
  e.oneshot_max_bytes = parse_env_int("CCL_ONESHOT_MAX_BYTES", -1);
  e.nvls = (int)parse_env_int("CCL_NVLS", 0);
  e.spin_timeout_ms = parse_env_int("CCL_SPIN_TIMEOUT_MS", -1);
  e.debug_bounds = parse_env_flag("CCL_DEBUG_BOUNDS", false);
  e.debug_checks = parse_env_flag("CCL_DEBUG_CHECKS", false);
  e.tune_file = env_str("CCL_TUNE_FILE", "");
  e.symm_mem = env_str("CCL_SYMM_MEM", "ipc");
  e.log_level = (int)parse_env_int("CCL_LOG_LEVEL", 0);
  e.arena_mb = parse_env_int("CCL_ARENA_MB", 256);
  e.symm_heap_mb = parse_env_int("CCL_SYMM_HEAP_MB", 1024);
  e.symm_min_bytes = parse_env_int("CCL_SYMM_MIN_BYTES", -1);
  e.nvls_min_bytes = parse_env_int("CCL_NVLS_MIN_BYTES", -1);
  e.round_mb = parse_env_int("CCL_ROUND_MB", -1);
  e.init_timeout_ms = parse_env_int("CCL_INIT_TIMEOUT_MS", -1);
  e.shm_slot_mb = parse_env_int("CCL_SHM_SLOT_MB", 4);
  e.max_blocks = (int)parse_env_int("CCL_MAX_BLOCKS", -1);
  e.threads = (int)parse_env_int("CCL_THREADS", -1);
  // launcher detection (reference: ProcessGroupCCL.cpp:825-830,930-945; dpcpp_ccl.cpp:137-152)
  e.with_mpirun = std::getenv("MPI_LOCALRANKID") || std::getenv("MPI_LOCALNRANKS") ||
                  std::getenv("PMI_RANK") || std::getenv("PMI_SIZE") || std::getenv("PMIX_RANK");
  e.local_rank = (int)parse_env_int("LOCAL_RANK", parse_env_int("MPI_LOCALRANKID", -1));
  e.local_world_size = (int)parse_env_int(
      "LOCAL_WORLD_SIZE", parse_env_int("MPI_LOCALNRANKS", parse_env_int("PALS_LOCAL_SIZE", -1)));
  return e;
}

}  // namespace

const Env& Env::get() {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_parsed) {
    g_env = parse();
    g_parsed = true;
  }
  return g_env;
}

void Env::reparse() {
  std::lock_guard<std::mutex> g(g_mu);
  g_env = parse();
  g_parsed = true;
}

}  // namespace ccl
