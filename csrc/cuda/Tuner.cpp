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

}  // namespace ccl
