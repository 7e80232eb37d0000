// Row-wise top-k selection by radix select, for the sparse-attention indexers (DeepSeek-V4 compressed-entry
// selection, GLM-DSA lightning indexer: top-512 / top-2048 of up to hundreds of thousands of scores per query row).
// One block per row: four 8-bit histogram passes over order-preserving integer keys find the k-th largest key, then
// one compaction pass writes the indices of everything above it and, in index order, as many ties as are still
// needed. The output is the index set in ascending index order (deterministic, lowest index wins a tie); entries
// beyond the number of selectable scores are -1. Scores equal to -inf are never selected.
// Reference counterpart: torch.topk in src/models/deepseek_v4/runtime.py (indexer) and the sort in
// src/models/glm_dsa/architecture.py:263-406; a sort of the whole row is replaced by five streaming passes.
#include "../common/pk_common.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float <=> larger key
}

struct TopkParams {
  const float* score;   // [M, ld]
  const int* length;    // [M] valid entries per row (null: n for every row)
  int n, ld, k;
  int* out;             // [M, k]
};

__global__ void __launch_bounds__(kThreads) topk_select_kernel(const TopkParams p) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_need, s_bucket;
  __shared__ uint32_t warp_tot[kThreads / 32][2];
  __shared__ uint32_t base[2];
  const int m = blockIdx.x, tid = threadIdx.x;
  const float* row = p.score + (size_t)m * p.ld;
  const int n = p.length ? min(max(p.length[m], 0), p.n) : p.n;
  int* out = p.out + (size_t)m * p.k;
  const uint32_t kNegInf = order_key(-INFINITY);

  // how many scores can be selected at all
  uint32_t prefix = 0, need = (uint32_t)p.k;   // keys with (key >> shift) > prefix are "above"; `need` of the bucket `prefix` remain
  // ---- four radix passes, most significant byte first ----
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kThreads) {
      const uint32_t key = order_key(row[i]);
      if (key == kNegInf) continue;
      // only keys that match the prefix found so far take part
      if (pass == 0 || (key >> (shift + 8)) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t acc = 0;
      int b = 255;
      for (; b >= 0; --b) {
        if (acc + hist[b] >= need) break;
        acc += hist[b];
      }
      if (b < 0) {          // fewer selectable scores than k: everything qualifies
        s_bucket = 0xffffffffu;
        s_need = 0;
      } else {
        s_bucket = (uint32_t)b;
        s_need = need - acc;   // still to take from bucket b
      }
    }
    __syncthreads();
    if (s_bucket == 0xffffffffu) {
      prefix = 0;
      need = 0;
      // threshold below everything: select all finite / non -inf scores
      break;
    }
    prefix = (prefix << 8) | s_bucket;
    need = s_need;
    __syncthreads();
  }
  const bool take_all = s_bucket == 0xffffffffu;
  // ---- compaction in index order: keys above the threshold, and the first `need` keys equal to it ----
  if (tid < 2) base[tid] = 0;
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  for (int i0 = 0; i0 < n; i0 += kThreads) {
    const int i = i0 + tid;
    bool above = false, equal = false;
    if (i < n) {
      const uint32_t key = order_key(row[i]);
      if (key != kNegInf) {
        above = take_all || key > prefix;
        equal = !take_all && key == prefix;
      }
    }
    const uint32_t ma = __ballot_sync(0xffffffffu, above), me = __ballot_sync(0xffffffffu, equal);
    if (lane == 0) {
      warp_tot[warp][0] = __popc(ma);
      warp_tot[warp][1] = __popc(me);
    }
    __syncthreads();
    uint32_t off_a = base[0], off_e = base[1];
    for (int w = 0; w < warp; ++w) {
      off_a += warp_tot[w][0];
      off_e += warp_tot[w][1];
    }
    const uint32_t lower = (1u << lane) - 1u;
    const uint32_t ra = off_a + __popc(ma & lower), re = off_e + __popc(me & lower);
    // final slot: ties that are taken interleave with the "above" set in index order, so the slot of an element is the
    // number of taken elements before it = above-before + min(equal-before, need)
    if (above) {
      const uint32_t slot = ra + min(re, need);
      if (slot < (uint32_t)p.k) out[slot] = i;
    } else if (equal && re < need) {
      const uint32_t slot = ra + re;
      if (slot < (uint32_t)p.k) out[slot] = i;
    }
    __syncthreads();
    if (tid == kThreads - 1) {
      base[0] = ra + (above ? 1u : 0u);
      base[1] = re + (equal ? 1u : 0u);
    }
    __syncthreads();
  }
  const uint32_t taken = base[0] + min(base[1], need);
  for (uint32_t s = taken + tid; s < (uint32_t)p.k; s += kThreads) out[s] = -1;
}

}  // namespace

// score fp32 [M, ld] (first n columns used), length [M] or null, out int32 [M, k]: indices of the k largest scores of
// each row in ascending index order, -1 padded.
PK_API int pk_topk_select(const float* score, const int* length, int M, int n, int ld, int k, int* out, cudaStream_t stream) {
  if (M < 1 || n < 1 || ld < n || k < 1) return PK_ERR_BAD_ARG;
  TopkParams p{score, length, n, ld, k, out};
  topk_select_kernel<<<M, kThreads, 0, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}
