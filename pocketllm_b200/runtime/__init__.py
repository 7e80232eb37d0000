"""Generation runtime: greedy loops, scheduling, prefix snapshots, speculative decoding."""
