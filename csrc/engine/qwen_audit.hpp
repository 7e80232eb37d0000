// Host-side audit of a Qwen hybrid checkpoint against its config: every tensor the engine will ask for must be there
// with the dtype and shape the shard rules assume, and every cut of the tensor-parallel split must fall on the 128-wide
// scale blocks of the FP8 linears. Nothing is uploaded; no GPU is needed. Role of the reference's `--qwen-audit`
// (cpp_engine/src/main.cpp:80-221, cpp_engine/src/qwen_weights.cpp shard rules).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "qwen_config.hpp"
#include "safetensors.hpp"

namespace pk {

struct QwenAuditReport {
  int expected = 0;                       // tensors the engine reads
  int fp8_linears = 0;
  uint64_t expected_bytes = 0;
  std::vector<std::string> problems;      // one line each: missing / dtype / shape / shard alignment
  std::vector<std::string> unused;        // tensors in the files that the engine never reads
  bool ok() const { return problems.empty(); }
};

// `want_mtp`: also require the multi-token predictor's tensors (mtp.*).
QwenAuditReport audit_qwen_checkpoint(const SafetensorsModel& st, const QwenConfig& cfg, int tp_world, bool want_mtp);

}  // namespace pk
