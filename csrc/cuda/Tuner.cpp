#include "cuda/Tuner.h"

#include <fstream>
#include <sstream>
#include <stdexcept>

namespace ccl {

namespace {

const char* const kKeys[] = {"oneshot_max_bytes", "ag_push_max_bytes", "max_blocks", "threads", "nvls_min_bytes", "symm_min_bytes", "round_bytes", "nvls_round_bytes", "ag_pull_round_bytes", "ag_nvls_max_bytes"};

bool known_key(const std::string& k) {
  for (const char* s : kKeys)
    if (k == s) return true;
  return false;
}

[[noreturn]] void fail(const std::string& path, int line, const std::string& what) {
  throw std::runtime_error("ccl: " + path + ":" + std::to_string(line) + ": " + what);
}

bool parse_ll(const std::string& s, long long* out) {
  if (s.empty()) return false;
  size_t pos = 0;
  try {
    *out = std::stoll(s, &pos, 10);
  } catch (...) {
    return false;
  }
  return pos == s.size();
}

}  // namespace

std::map<int, TuneEntry> parse_tune_text(const std::string& text, const std::string& path) {
  std::map<int, TuneEntry> table;
  std::istringstream in(text);
  std::string line;
  int ln = 0;
  while (std::getline(in, line)) {
    ++ln;
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.resize(hash);
    std::istringstream ls(line);
    std::string tok;
    if (!(ls >> tok)) continue;
    long long world = 0;
    if (!parse_ll(tok, &world) || world < 1 || world > kMaxRanks) fail(path, ln, "expected a world size 1.." + std::to_string(kMaxRanks) + ", got '" + tok + "'");
    if (table.count((int)world)) fail(path, ln, "world size " + tok + " appears twice");
    TuneEntry e;
    while (ls >> tok) {
      const size_t eq = tok.find('=');
      if (eq == std::string::npos) fail(path, ln, "expected key=value, got '" + tok + "'");
      const std::string k = tok.substr(0, eq);
      long long v = 0;
      if (!known_key(k)) fail(path, ln, "unknown key '" + k + "'");
      if (!parse_ll(tok.substr(eq + 1), &v) || v < 0) fail(path, ln, "value of '" + k + "' must be a non-negative integer");
      if ((k == "max_blocks" && (v < 1 || v > kMaxBlocks)) || (k == "threads" && (v < 32 || v > 512 || v % 32)))
        fail(path, ln, "value of '" + k + "' out of range");
      e[k] = v;
    }
    if (e.empty()) fail(path, ln, "no key=value pairs");
    table[(int)world] = e;
  }
  return table;
}

std::map<int, TuneEntry> parse_tune_file(const std::string& path) {
  std::ifstream f(path);
  if (!f) throw std::runtime_error("ccl: cannot open CCL_TUNE_FILE '" + path + "'");
  std::stringstream ss;
  ss << f.rdbuf();
  return parse_tune_text(ss.str(), path);
}

bool apply_tuning(const std::map<int, TuneEntry>& table, int world, CommConfig* cfg) {
  auto it = table.find(world);
  if (it == table.end()) return false;
  for (const auto& kv : it->second) {
    if (kv.first == "oneshot_max_bytes") cfg->oneshot_max_bytes = (size_t)kv.second;
    else if (kv.first == "ag_push_max_bytes") cfg->ag_push_max_bytes = (size_t)kv.second;
    else if (kv.first == "max_blocks") cfg->max_blocks = (int)kv.second;
    else if (kv.first == "threads") cfg->threads = (int)kv.second;
    else if (kv.first == "nvls_min_bytes") cfg->nvls_min_bytes = (size_t)kv.second;
    else if (kv.first == "symm_min_bytes") cfg->symm_min_bytes = (size_t)kv.second;
    else if (kv.first == "round_bytes") cfg->round_bytes = (size_t)kv.second;
    else if (kv.first == "nvls_round_bytes") cfg->nvls_round_bytes = (size_t)kv.second;
    else if (kv.first == "ag_pull_round_bytes") cfg->ag_pull_round_bytes = (size_t)kv.second;
    else if (kv.first == "ag_nvls_max_bytes") cfg->ag_nvls_max_bytes = (size_t)kv.second;
  }
  return true;
}

// Built-in thresholds for the knobs left at "-1", from `bench/tune.py` and `bench/sweep.py` on B200 + NVSwitch:
//  * zero-copy path for symmetric tensors: from 512 KB at 8 ranks (16.9 vs 18.7 us), 2 MB at 4 ranks (18.2 vs 25.8 us;
//    below it the staged one-shot kernel is 1-3 us faster), 16 MB at 2 ranks (nothing to save with one peer);
//  * staged switch (NVLS) kernels: from 2 MB at 8 ranks (28 vs 40 us), 8 MB at 4 ranks (44.5 vs 58 us; two-shot wins at
//    4 MB, 30 vs 34 us), never at 2 ranks (512 MB: all_reduce 1736 vs 1320 us, reduce_scatter 1045 vs 786, all_gather
//    893 vs 510 - with one peer the switch saves no NVLink bytes);
//  * staging rounds: 128 MB for the peer-memory kernels (512 MB bf16 at 2 / 4 ranks: all_reduce 1320 -> 1202 / 1635 ->
//    1532 us, reduce_scatter 786 -> 731 / 927 -> 879, all_to_all 680 -> 643 / 819 -> 798; 64 MB and 32 MB are slower),
//    64 MB for the switch kernels (4 ranks: all_reduce 1522 -> 1417 us, reduce_scatter 904 -> 844 against 128 MB rounds;
//    8 ranks against rounds of the whole 256 MB arena half: all_reduce 1533 -> 1305 us, reduce_scatter 923 -> 835,
//    all_gather 809 -> 783 with its outputs >= 128 MB on the pull mode in 32 MB rounds).
void resolve_builtin_thresholds(int world, CommConfig* cfg) {
  if (cfg->symm_min_bytes == (size_t)-1) cfg->symm_min_bytes = world <= 2 ? (16u << 20) : world <= 4 ? (2u << 20) : (512u << 10);
  if (cfg->nvls_min_bytes == (size_t)-1) cfg->nvls_min_bytes = world <= 2 ? ((size_t)1 << 62) : world <= 4 ? (8u << 20) : (2u << 20);
  if (cfg->nvls_round_bytes == (size_t)-1) cfg->nvls_round_bytes = cfg->round_bytes != (size_t)-1 ? cfg->round_bytes : (64u << 20);
  if (cfg->ag_pull_round_bytes == (size_t)-1) cfg->ag_pull_round_bytes = cfg->round_bytes != (size_t)-1 ? cfg->round_bytes : (32u << 20);
  if (cfg->round_bytes == (size_t)-1) cfg->round_bytes = 128u << 20;
}

}  // namespace ccl
