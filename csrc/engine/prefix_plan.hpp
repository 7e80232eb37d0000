// Host-side decisions of exact prefix reuse across sequential requests of the hybrid decoder.
//
// The full-attention KV cache is indexed by position and survives between requests, so a new prompt that shares its
// first L tokens with what the engine has already consumed needs no attention work for them. The recurrent DeltaNet
// state is NOT indexed by position: it can be continued from where it stands ("live": the new prompt extends the whole
// consumed sequence) or rolled back to a stored copy taken at some position <= L ("snapshot"), else the request starts
// from zero ("empty"). Positions past the resume point are overwritten by the new request, so snapshots taken beyond it
// die. Behavioural counterpart: cpp_engine/src/qwen_engine.cpp:662-826 and 1979-2149 of the reference
// (prefix_cache, state_snapshot_interval_tokens, max_state_snapshots).
#pragma once

#include <algorithm>
#include <string>
#include <vector>

namespace pk {

struct PrefixDecision {
  enum Source { kEmpty = 0, kLive = 1, kSnapshot = 2 };
  Source source = kEmpty;
  int resume_pos = 0;      // tokens of the new prompt that need no forward pass
  int snapshot_index = -1; // into the positions passed to plan_prefix (kSnapshot only)
  int matched = 0;         // common prefix with the consumed sequence, before rounding to a resume point
};

inline const char* prefix_source_name(PrefixDecision::Source s) {
  return s == PrefixDecision::kLive ? "live" : s == PrefixDecision::kSnapshot ? "snapshot" : "empty";
}

// `history`: tokens consumed so far (positions 0 .. live_pos-1 hold valid KV and the recurrent state stands at
// live_pos). `snapshot_pos`: positions of the stored recurrent states (each <= live_pos when it was taken).
// At least one prompt token is always left to run, because the request needs the logits of its last token.
inline PrefixDecision plan_prefix(const std::vector<int>& history, int live_pos, const std::vector<int>& snapshot_pos,
                                  const int* prompt, int n) {
  PrefixDecision d;
  const int lim = std::min<int>({(int)history.size(), live_pos, n});
  int l = 0;
  while (l < lim && history[(size_t)l] == prompt[l]) ++l;
  d.matched = l;
  const int usable = std::min(l, n - 1);
  if (usable <= 0) return d;
  if (l == live_pos && live_pos <= n - 1) {   // the prompt continues exactly where the engine stands
    d.source = PrefixDecision::kLive;
    d.resume_pos = live_pos;
    return d;
  }
  int best = -1;
  for (size_t i = 0; i < snapshot_pos.size(); ++i)
    if (snapshot_pos[i] > 0 && snapshot_pos[i] <= usable && (best < 0 || snapshot_pos[i] > snapshot_pos[(size_t)best])) best = (int)i;
  if (best >= 0) {
    d.source = PrefixDecision::kSnapshot;
    d.resume_pos = snapshot_pos[(size_t)best];
    d.snapshot_index = best;
  }
  return d;
}

// Positions at which a prefill from `from` to `to` stores the recurrent state: every multiple of `interval` inside
// (from, to), plus `to` itself (the request boundary). interval <= 0: only the boundary.
inline std::vector<int> snapshot_points(int from, int to, int interval) {
  std::vector<int> pts;
  if (interval > 0)
    for (int p = (from / interval + 1) * interval; p < to; p += interval) pts.push_back(p);
  if (to > from) pts.push_back(to);
  return pts;
}

// Which stored snapshot to drop when the store is full: the oldest one that is not a multiple of the interval
// (request boundaries are the most specific), else the oldest.
inline int snapshot_to_evict(const std::vector<int>& snapshot_pos, const std::vector<long long>& stamp, int interval) {
  int victim = -1;
  for (size_t i = 0; i < snapshot_pos.size(); ++i) {
    const bool boundary = interval <= 0 || snapshot_pos[i] % interval != 0;
    if (!boundary) continue;
    if (victim < 0 || stamp[i] < stamp[(size_t)victim]) victim = (int)i;
  }
  if (victim >= 0) return victim;
  for (size_t i = 0; i < snapshot_pos.size(); ++i)
    if (victim < 0 || stamp[i] < stamp[(size_t)victim]) victim = (int)i;
  return victim;
}

}  // namespace pk
