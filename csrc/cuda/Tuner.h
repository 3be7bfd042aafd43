// Per-world-size tuning of the CUDA collectives, read from the text file that CCL_TUNE_FILE
// names and that `bench/tune.py` writes from measurements on the machine at hand.
//
// Format: one line per world size, `#` starts a comment:
//     <world> key=value [key=value ...]
// keys: oneshot_max_bytes, ag_push_max_bytes (0 = built-in default, 1 = never), max_blocks, threads. Unknown keys and malformed
// lines are errors (a silently ignored tuning file is worse than none). Environment variables
// that set the same knob explicitly win over the file.
//
// The reference hard-codes its thresholds (one-shot up to 458 752 fp16 elements, chunking at
// 32 Mi elements: src/gpu/allreduce_small.h:24, src/gpu/allreduce.h:33); there is no tuner.
#pragma once
#include <map>
#include <string>

#include "cuda/CudaComm.h"

namespace ccl {

using TuneEntry = std::map<std::string, long long>;

// Parses the whole file: world size -> {key: value}. Throws std::runtime_error with
// "<path>:<line>: ..." on any problem.
std::map<int, TuneEntry> parse_tune_text(const std::string& text, const std::string& path_for_messages);
std::map<int, TuneEntry> parse_tune_file(const std::string& path);

// Applies the line for `world` (if any) to `cfg`; returns true when a line matched.
bool apply_tuning(const std::map<int, TuneEntry>& table, int world, CommConfig* cfg);

// Replaces every threshold of `cfg` that is still at its "-1 = built-in" value by the measured default for `world` ranks.
void resolve_builtin_thresholds(int world, CommConfig* cfg);

}  // namespace ccl
