// Plain-C descriptions of one collective "site" of the peer-memory protocol, shared by
// host code (which fills them) and device code (which acts on them).
#pragma once

#include <stdint.h>

#define PK_MAX_RANKS 8

// One collective "site": where a producer pushes and how it signals.
struct PkPush {
  float* dst[PK_MAX_RANKS];      // peer r's slot buffer base ([world][rows][cols] fp32)
  uint32_t* flag[PK_MAX_RANKS];  // peer r's flag array base ([world] words for this slot)
  uint32_t* block_counter;       // local, zero between launches
  const uint32_t* epoch;         // local device word, bumped once per forward
  uint32_t sites_per_epoch;
  uint32_t site;
  int world;
  int rank;
  // Reduce-scatter form (prefill GEMM epilogues): rows are owned in blocks of `rows_per_rank`; row m goes ONLY to rank
  // m / rows_per_rank, at row (rank * rows_per_rank + m % rows_per_rank) of its slot [world][rows_per_rank][cols].
  // 0 = every row to every rank (slot [world][rows][cols]).
  int rows_per_rank;
};

// What a consumer waits on before reading its local slot buffer.
struct PkWait {
  const uint32_t* flag;   // local flag array base ([world] words for this slot), or null
  const uint32_t* epoch;  // local device word
  uint32_t sites_per_epoch;
  uint32_t site;
  int world;
  uint32_t* status;       // local status word, 0 = ok
  uint32_t timeout_us;
};

#define PK_COMM_TIMEOUT 1u
// another rank reported a timeout in the same step (learned through the sampler exchange)
#define PK_COMM_PEER_FAILED 4u

