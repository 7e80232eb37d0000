// Draft-length policy of speculative decode, kept apart from the engine so that the host self-test can exercise it:
// start at one draft, double after a fully accepted round up to the limit, and after a reject fall back to
// max(1, min(K / 2, accepted + 1)) (reference: cpp_engine/src/qwen_engine.cpp:2169-2270).
#pragma once

#include <algorithm>

namespace pk {

// K: the current draft length; used: drafts actually sent this round (<= K, fewer near the end of a request);
// accepted: how many of them the target matched.
inline int next_draft_len(int K, int used, int accepted, int max_draft) {
  if (accepted >= used) return std::min(2 * K, std::max(1, max_draft));
  return std::max(1, std::min(K / 2, accepted + 1));
}

// Drafts to send when `remaining` tokens are still wanted: the last token of a request always comes from a plain step.
inline int drafts_this_round(int K, int remaining, int max_draft) {
  return std::max(0, std::min(K, std::min(remaining - 1, max_draft)));
}

}  // namespace pk
