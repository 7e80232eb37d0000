// C ABI of the native engine, used by the Python package (ctypes) and by external
// callers. Every function returns 0 on success; pk_engine_last_error() gives the
// message of the last failure on the calling thread.
#include <algorithm>
#include <cstring>
#include <string>

#include "json.hpp"
#include "gguf_reader.hpp"
#include "mem_guard.hpp"
#include "qwen_engine.hpp"
#include "sampler.hpp"
#include "kv_swap.hpp"
#include "staging.hpp"
#include "tokenizer.hpp"

#define PK_EAPI extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_err;

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown error";
    return 1;
  }
}
}  // namespace

// Decision of the device-memory floor (POCKET_MIN_FREE_MIB) for given numbers: 0 and an empty message when the request
// fits, 1 and the refusal text otherwise.
PK_EAPI int pk_mem_headroom_verdict(unsigned long long free_bytes, unsigned long long total_bytes, unsigned long long request_bytes,
                                    unsigned long long min_free_bytes, char* msg, int msg_len) {
  const std::string m = pk::headroom_verdict(free_bytes, total_bytes, request_bytes, min_free_bytes, "request");
  if (msg && msg_len > 0) std::snprintf(msg, (size_t)msg_len, "%s", m.c_str());
  return m.empty() ? 0 : 1;
}

PK_EAPI const char* pk_engine_last_error() { return g_err.c_str(); }

// config_json: a Hugging Face style config (flat or under text_config), or the literal
// "benchmark_27b" for the 64-layer benchmark shape.
PK_EAPI void* pk_qwen_create_ex(const char* config_json, int tp_rank, int tp_world, int device, int max_context,
                                int prefill_chunk, int use_cuda_graph, int decode_splits, int mtp);
PK_EAPI void* pk_qwen_create_ex2(const char* config_json, int tp_rank, int tp_world, int device, int max_context,
                                 int prefill_chunk, int use_cuda_graph, int decode_splits, int mtp, int kv_fp8);

PK_EAPI void* pk_qwen_create(const char* config_json, int tp_rank, int tp_world, int device, int max_context,
                             int prefill_chunk, int use_cuda_graph, int decode_splits) {
  return pk_qwen_create_ex(config_json, tp_rank, tp_world, device, max_context, prefill_chunk, use_cuda_graph, decode_splits, 0);
}

// mtp != 0 also builds the multi-token predictor (`mtp.*` tensors) used by pk_qwen_spec_decode.
PK_EAPI void* pk_qwen_create_ex(const char* config_json, int tp_rank, int tp_world, int device, int max_context,
                                int prefill_chunk, int use_cuda_graph, int decode_splits, int mtp) {
  return pk_qwen_create_ex2(config_json, tp_rank, tp_world, device, max_context, prefill_chunk, use_cuda_graph, decode_splits, mtp, 0);
}

// kv_fp8 != 0: FP8 KV cache (E4M3 codes, one scale per 64 channels) instead of bf16.
PK_EAPI void* pk_qwen_create_ex2(const char* config_json, int tp_rank, int tp_world, int device, int max_context,
                                 int prefill_chunk, int use_cuda_graph, int decode_splits, int mtp, int kv_fp8) {
  pk::QwenEngine* eng = nullptr;
  guarded([&] {
    pk::QwenConfig cfg = std::string(config_json) == "benchmark_27b"
                             ? pk::QwenConfig::benchmark_27b()
                             : pk::QwenConfig::from_json(pk::Json::parse(std::string(config_json)));
    pk::QwenEngineOptions opt;
    opt.tp_rank = tp_rank;
    opt.tp_world = tp_world;
    opt.device = device;
    if (max_context > 0) opt.max_context = max_context;
    if (prefill_chunk > 0) opt.prefill_chunk = prefill_chunk;
    // 0 = choose from the context length: one split per 2048 positions, between 8 and 64
    if (decode_splits > 0) opt.decode_splits = decode_splits;
    else opt.decode_splits = std::min(64, std::max(8, max_context / 2048));
    opt.use_cuda_graph = use_cuda_graph != 0;
    opt.mtp = mtp != 0;
    opt.kv_fp8 = kv_fp8 != 0;
    eng = new pk::QwenEngine(cfg, opt);
  });
  return eng;
}

PK_EAPI void pk_qwen_destroy(void* h) { delete (pk::QwenEngine*)h; }

PK_EAPI int pk_qwen_load_safetensors(void* h, const char* path) {
  return guarded([&] { ((pk::QwenEngine*)h)->load_safetensors(path); });
}

PK_EAPI int pk_qwen_init_random(void* h, uint64_t seed, float sigma) {
  return guarded([&] { ((pk::QwenEngine*)h)->init_random(seed, sigma); });
}

PK_EAPI int pk_qwen_reset(void* h) {
  return guarded([&] { ((pk::QwenEngine*)h)->reset(); });
}

PK_EAPI int pk_qwen_prefill(void* h, const int* tokens, int n, int* first_token) {
  return guarded([&] {
    const int t = ((pk::QwenEngine*)h)->prefill(tokens, n);
    if (first_token) *first_token = t;
  });
}

// A new request with exact prefix reuse (see prefix_plan.hpp). stats (may be null): [reused, computed, prompt, matched,
// source (0 empty, 1 live, 2 snapshot), snapshots, snapshot_bytes, hits, misses].
PK_EAPI int pk_qwen_prefill_cached(void* h, const int* tokens, int n, int* first_token, long long* stats) {
  return guarded([&] {
    auto* e = (pk::QwenEngine*)h;
    const int t = e->prefill_cached(tokens, n);
    if (first_token) *first_token = t;
    if (stats) {
      const pk::QwenPrefixStats& ps = e->prefix_stats();
      const std::string src = ps.resume_source;
      const long long v[9] = {ps.reused_tokens, ps.computed_tokens, ps.prompt_tokens, ps.matched_tokens,
                              src == "live" ? 1 : src == "snapshot" ? 2 : 0, ps.snapshots, (long long)ps.snapshot_bytes, ps.hits, ps.misses};
      for (int i = 0; i < 9; ++i) stats[i] = v[i];
    }
  });
}
// interval 0: recurrent-state copies at request boundaries only; max_snapshots 0: live continuation only; enable 0: off.
PK_EAPI int pk_qwen_configure_prefix_cache(void* h, int enable, int snapshot_interval, int max_snapshots) {
  return guarded([&] { ((pk::QwenEngine*)h)->configure_prefix_cache(enable != 0, snapshot_interval, max_snapshots); });
}
PK_EAPI int pk_qwen_clear_prefix_cache(void* h) {
  return guarded([&] { ((pk::QwenEngine*)h)->clear_prefix_cache(); });
}

PK_EAPI int pk_qwen_decode(void* h, int steps, int* out_tokens, int sync_each_step) {
  return guarded([&] { ((pk::QwenEngine*)h)->decode(steps, out_tokens, sync_each_step != 0); });
}

PK_EAPI int pk_qwen_forward_rows(void* h, const int* tokens, int M, int* out_tokens) {
  return guarded([&] { ((pk::QwenEngine*)h)->forward_rows(tokens, M, out_tokens); });
}

// Speculative greedy decode with the multi-token predictor; the tokens equal those of pk_qwen_decode.
// stats (may be null): [rounds, proposed, accepted, rollbacks, replay_tokens, plain_steps, predictor_rows].
PK_EAPI int pk_qwen_spec_decode(void* h, int steps, int max_draft, int* out_tokens, long long* stats) {
  return guarded([&] {
    pk::QwenSpecStats st;
    ((pk::QwenEngine*)h)->spec_decode(steps, max_draft, out_tokens, &st);
    if (stats) {
      const long long v[7] = {st.rounds, st.proposed, st.accepted, st.rollbacks, st.replay_tokens, st.plain_steps, st.predictor_rows};
      for (int i = 0; i < 7; ++i) stats[i] = v[i];
    }
  });
}
PK_EAPI int pk_qwen_mtp_next_token(void* h) { return ((pk::QwenEngine*)h)->mtp_next_token(); }
PK_EAPI int pk_qwen_copy_mtp_logits(void* h, float* out) {
  return guarded([&] { ((pk::QwenEngine*)h)->copy_mtp_logits(out); });
}
PK_EAPI int pk_qwen_mtp_enabled(void* h) { return ((pk::QwenEngine*)h)->mtp_enabled() ? 1 : 0; }
// Test hook: drafts are taken from this continuation (the tokens that follow the first generated one); n = 0 clears it.
PK_EAPI int pk_qwen_set_draft_replay(void* h, const int* tokens, int n) {
  return guarded([&] { ((pk::QwenEngine*)h)->set_draft_replay(tokens, n); });
}

// Recurrent-state snapshots (KV is position indexed and is not copied). A snapshot handle
// belongs to the engine that made it.
PK_EAPI void* pk_qwen_snapshot(void* h) {
  void* out = nullptr;
  guarded([&] { out = ((pk::QwenEngine*)h)->snapshot().release(); });
  return out;
}
// Snapshot that also holds the KV rows of positions [0, position): survives other requests (prefix cache).
PK_EAPI void* pk_qwen_snapshot_with_kv(void* h) {
  void* out = nullptr;
  guarded([&] { out = ((pk::QwenEngine*)h)->snapshot(true).release(); });
  return out;
}
PK_EAPI int pk_qwen_snapshot_update(void* h, void* snap) {
  return guarded([&] { ((pk::QwenEngine*)h)->update_snapshot(*(pk::QwenEngine::Snapshot*)snap); });
}
PK_EAPI int pk_qwen_restore(void* h, void* snap) {
  return guarded([&] { ((pk::QwenEngine*)h)->restore(*(pk::QwenEngine::Snapshot*)snap); });
}
PK_EAPI int pk_qwen_snapshot_position(void* snap) { return ((pk::QwenEngine::Snapshot*)snap)->pos; }
PK_EAPI int pk_qwen_free_snapshot(void* h, void* snap) {
  return guarded([&] {
    auto* s = (pk::QwenEngine::Snapshot*)snap;
    ((pk::QwenEngine*)h)->free_snapshot(*s);
    delete s;
  });
}

PK_EAPI int pk_qwen_copy_logits(void* h, float* out, int row) {
  return guarded([&] { ((pk::QwenEngine*)h)->copy_logits(out, row); });
}

// 1 when single-row decode steps run on the persistent whole-token kernel (known after the first decode call).
PK_EAPI int pk_qwen_persistent_decode_active(void* h) { return ((pk::QwenEngine*)h)->persistent_decode_active() ? 1 : 0; }

PK_EAPI int pk_qwen_set_persistent_decode(void* h, int mode) {
  return guarded([&] { ((pk::QwenEngine*)h)->set_persistent_decode(mode); });
}

// mode as QwenEngineOptions::prefill_gemm; call before loading or initialising the weights
PK_EAPI int pk_qwen_set_prefill_gemm(void* h, int mode) {
  return guarded([&] { ((pk::QwenEngine*)h)->set_prefill_gemm(mode); });
}
PK_EAPI int pk_qwen_prefill_gemm_mode(void* h) { return ((pk::QwenEngine*)h)->prefill_gemm_mode(); }

PK_EAPI int pk_qwen_enable_nccl_fallback(void* h, const char* id_path, int timeout_ms) {
  return guarded([&] { ((pk::QwenEngine*)h)->enable_nccl_fallback(id_path, timeout_ms > 0 ? timeout_ms : 600000); });
}
PK_EAPI int pk_qwen_switch_to_nccl(void* h) {
  return guarded([&] { ((pk::QwenEngine*)h)->switch_to_nccl(); });
}
PK_EAPI int pk_qwen_nccl_mode(void* h) { return ((pk::QwenEngine*)h)->nccl_mode() ? 1 : 0; }
PK_EAPI int pk_qwen_set_comm_timeout_us(void* h, unsigned us) {
  return guarded([&] { ((pk::QwenEngine*)h)->set_comm_timeout_us(us); });
}

// -1: every guard intact (or canaries off); else the index of the damaged buffer, described in pk_engine_last_error()
PK_EAPI int pk_qwen_verify_canaries(void* h) {
  int idx = -1;
  std::string what;
  if (guarded([&] { idx = ((pk::QwenEngine*)h)->verify_canaries(&what); }) != 0) return -2;
  if (idx >= 0) g_err = what;
  return idx;
}
PK_EAPI int pk_qwen_canaries_enabled(void* h) { return ((pk::QwenEngine*)h)->canaries_enabled() ? 1 : 0; }

PK_EAPI int pk_qwen_set_tap_layers(void* h, const int* layers, int n) {
  return guarded([&] { ((pk::QwenEngine*)h)->set_tap_layers(layers, n); });
}
PK_EAPI int pk_qwen_tap_rows(void* h) { return ((pk::QwenEngine*)h)->tap_rows(); }
// rows [first_row, first_row + rows) of the last forward's taps, [rows, taps * hidden] bf16, into device memory
PK_EAPI int pk_qwen_copy_taps(void* h, void* dst_device, int first_row, int rows) {
  return guarded([&] { ((pk::QwenEngine*)h)->copy_taps(dst_device, first_row, rows); });
}

PK_EAPI int pk_qwen_decode_trace(void* h, unsigned long long* out, int cap) {
  int n = 0;
  guarded([&] { n = ((pk::QwenEngine*)h)->copy_decode_trace(out, cap); });
  return n;
}

PK_EAPI int pk_qwen_vocab_local(void* h) { return ((pk::QwenEngine*)h)->vocab_local(); }
PK_EAPI int pk_qwen_position(void* h) { return ((pk::QwenEngine*)h)->position(); }
PK_EAPI int pk_qwen_last_token(void* h) { return ((pk::QwenEngine*)h)->last_token(); }
PK_EAPI unsigned pk_qwen_comm_status(void* h) {
  unsigned s = 0xffffffffu;
  guarded([&] { s = ((pk::QwenEngine*)h)->comm_status(); });
  return s;
}
PK_EAPI unsigned long long pk_qwen_kv_cache_bytes(void* h) { return ((pk::QwenEngine*)h)->kv_cache_bytes(); }
PK_EAPI unsigned long long pk_qwen_weight_bytes(void* h) { return ((pk::QwenEngine*)h)->weight_bytes(); }
// bytes of the bf16 copies kept for the prefill GEMM (0 when they are off)
PK_EAPI unsigned long long pk_qwen_shadow_bytes(void* h) { return ((pk::QwenEngine*)h)->shadow_bytes(); }

// out[0] prefill_ms, out[1] decode_ms, out[2] prefill_tokens, out[3] decode_tokens, out[4] launches
PK_EAPI void pk_qwen_timings(void* h, double* out) {
  const pk::QwenTimings& t = ((pk::QwenEngine*)h)->timings();
  out[0] = t.prefill_ms;
  out[1] = t.decode_ms;
  out[2] = t.prefill_tokens;
  out[3] = t.decode_tokens;
  out[4] = (double)t.kernel_launches;
}

// ---- peer memory plumbing (handles travel through the host control plane) ----
PK_EAPI void* pk_qwen_comm_arena(void* h, unsigned long long* bytes) {
  auto* e = (pk::QwenEngine*)h;
  if (bytes) *bytes = e->comm_arena_bytes();
  return e->comm_arena();
}

PK_EAPI int pk_qwen_set_peer_arenas(void* h, void* const* arenas) {
  return guarded([&] { ((pk::QwenEngine*)h)->set_peer_arenas(arenas); });
}

PK_EAPI int pk_ipc_export(void* dev_ptr, void* handle_out_64) {
  return guarded([&] {
    cudaIpcMemHandle_t hd;
    cudaError_t e = cudaIpcGetMemHandle(&hd, dev_ptr);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    static_assert(sizeof(hd) == 64, "ipc handle size");
    memcpy(handle_out_64, &hd, 64);
  });
}

PK_EAPI void* pk_ipc_open(const void* handle_64) {
  void* p = nullptr;
  guarded([&] {
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle_64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
  });
  return p;
}

PK_EAPI int pk_ipc_close(void* p) {
  return guarded([&] {
    cudaError_t e = cudaIpcCloseMemHandle(p);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaIpcCloseMemHandle: ") + cudaGetErrorString(e));
  });
}

// Host sampler (greedy when temperature <= 0). `rng_state` is advanced in place and must be non-zero.
PK_EAPI int pk_sample_token(const float* logits, int n, float temperature, float top_p, int top_k, uint64_t* rng_state) {
  pk::SamplerConfig c;
  c.temperature = temperature;
  c.top_p = top_p;
  c.top_k = top_k;
  return pk::sample_token(logits, n, c, *rng_state);
}

// Native GGUF reader: returns the metadata plus the tensor table as a JSON string owned by the
// calling thread (valid until its next call), or null on error.
PK_EAPI const char* pk_gguf_describe(const char* path) {
  thread_local std::string out;
  const int rc = guarded([&] {
    pk::GgufFile f(path);
    pk::Json j = pk::Json::object();
    j["version"] = pk::Json((int64_t)f.version());
    j["alignment"] = pk::Json((int64_t)f.alignment());
    j["metadata"] = f.metadata();
    pk::Json ts = pk::Json::array();
    for (const auto& t : f.tensors()) {
      pk::Json e = pk::Json::object();
      e["name"] = pk::Json(t.name);
      e["type"] = pk::Json(pk::ggml_type_name(t.type));
      pk::Json dims = pk::Json::array();
      for (uint64_t d : t.dims) dims.push_back(pk::Json((int64_t)d));
      e["dims"] = dims;
      e["offset"] = pk::Json((int64_t)t.offset);
      e["nbytes"] = pk::Json((int64_t)t.nbytes);
      // first bytes of the data, so that callers can check the mapping
      const uint8_t* p = f.data(t);
      int64_t sum = 0;
      for (uint64_t i = 0; i < (t.nbytes < 64 ? t.nbytes : 64); ++i) sum += p[i];
      e["head_sum"] = pk::Json(sum);
      ts.push_back(e);
    }
    j["tensors"] = ts;
    out = j.dump();
  });
  return rc == 0 ? out.c_str() : nullptr;
}

// Native byte-level BPE tokenizer from a GGUF file's metadata.
PK_EAPI void* pk_tokenizer_from_gguf(const char* path) {
  void* out = nullptr;
  guarded([&] {
    pk::GgufFile f(path);
    out = new pk::BpeTokenizer(pk::BpeTokenizer::from_gguf(f));
  });
  return out;
}
// ... or from a Hugging Face tokenizer directory / tokenizer.json file.
PK_EAPI void* pk_tokenizer_from_hf(const char* dir_or_file) {
  void* out = nullptr;
  guarded([&] { out = new pk::BpeTokenizer(pk::BpeTokenizer::from_hf_dir(dir_or_file)); });
  return out;
}
PK_EAPI void pk_tokenizer_destroy(void* t) { delete (pk::BpeTokenizer*)t; }
// Writes up to `cap` ids; returns the number of ids of the full encoding (call again with a larger buffer if > cap), -1 on error.
PK_EAPI int pk_tokenizer_encode(void* t, const char* text, int parse_special, int* out, int cap) {
  int n = -1;
  guarded([&] {
    const std::vector<int> ids = ((pk::BpeTokenizer*)t)->encode(text, parse_special != 0);
    for (int i = 0; i < (int)ids.size() && i < cap; ++i) out[i] = ids[i];
    n = (int)ids.size();
  });
  return n;
}
// UTF-8 text owned by the calling thread (valid until its next call); null on error.
PK_EAPI const char* pk_tokenizer_decode(void* t, const int* ids, int n, int skip_special) {
  thread_local std::string text;
  const int rc = guarded([&] { text = ((pk::BpeTokenizer*)t)->decode(std::vector<int>(ids, ids + n), skip_special != 0); });
  return rc == 0 ? text.c_str() : nullptr;
}

// ---- host-to-device expert staging -----------------------------------------------------------------------------------

// ---- KV swap tier ----
PK_EAPI void* pk_kvswap_create(int capacity, int device_slots, unsigned long long row_bytes, int window, int host_only) {
  void* out = nullptr;
  guarded([&] { out = new pk::KvSwapTier(capacity, device_slots, (size_t)row_bytes, window, host_only != 0); });
  return out;
}
PK_EAPI void pk_kvswap_destroy(void* h) { delete (pk::KvSwapTier*)h; }
PK_EAPI int pk_kvswap_store(void* h, int first, int count, const void* rows_device, void* stream) {
  return guarded([&] { ((pk::KvSwapTier*)h)->store(first, count, rows_device, (cudaStream_t)stream); });
}
PK_EAPI int pk_kvswap_swap_in(void* h, const int* selected_device, int n, void* pool_device, int* physical_device, void* stream) {
  return guarded([&] { ((pk::KvSwapTier*)h)->swap_in(selected_device, n, pool_device, physical_device, (cudaStream_t)stream); });
}
PK_EAPI int pk_kvswap_reset(void* h) {
  return guarded([&] { ((pk::KvSwapTier*)h)->reset(); });
}
// out[0] hits, [1] misses, [2] h2d bytes, [3] d2h bytes, [4] evictions, [5] steps, [6] stored rows, [7] host bytes
PK_EAPI void pk_kvswap_stats(void* h, unsigned long long* out) {
  const pk::KvSwapTier* t = (const pk::KvSwapTier*)h;
  const pk::KvSwapStats& s = t->stats();
  out[0] = s.hits; out[1] = s.misses; out[2] = s.h2d_bytes; out[3] = s.d2h_bytes; out[4] = s.evictions; out[5] = s.steps;
  out[6] = (unsigned long long)t->stored_rows(); out[7] = (unsigned long long)t->host_bytes();
}

PK_EAPI void* pk_lru_create(int slots) {
  pk::LruSlotMap* m = nullptr;
  guarded([&] { m = new pk::LruSlotMap(slots); });
  return m;
}
PK_EAPI void pk_lru_destroy(void* h) { delete (pk::LruSlotMap*)h; }
// out_slots[n]; load_keys / load_slots receive up to n entries, *n_loads their count; stats = {hits, misses, evictions}.
PK_EAPI int pk_lru_assign(void* h, const long long* keys, int n, int* out_slots, long long* load_keys, int* load_slots, int* n_loads,
                          long long* stats) {
  return guarded([&] {
    auto* m = (pk::LruSlotMap*)h;
    std::vector<std::pair<long long, int>> loads;
    const std::vector<int> slots = m->assign(std::vector<long long>(keys, keys + n), &loads);
    for (int i = 0; i < n; ++i) out_slots[i] = slots[i];
    for (size_t i = 0; i < loads.size(); ++i) {
      load_keys[i] = loads[i].first;
      load_slots[i] = loads[i].second;
    }
    *n_loads = (int)loads.size();
    if (stats) {
      stats[0] = m->hits;
      stats[1] = m->misses;
      stats[2] = m->evictions;
    }
  });
}

PK_EAPI void* pk_expert_arena_create(int device_slots, unsigned long long expert_bytes, int ring_slots) {
  pk::ExpertSlotArena* a = nullptr;
  guarded([&] { a = new pk::ExpertSlotArena(device_slots, (size_t)expert_bytes, ring_slots); });
  return a;
}
PK_EAPI void pk_expert_arena_destroy(void* h) { delete (pk::ExpertSlotArena*)h; }
PK_EAPI int pk_expert_arena_set_host_store(void* h, const void* base, long long n_experts) {
  return guarded([&] { ((pk::ExpertSlotArena*)h)->set_host_store(base, n_experts); });
}
// stats = {hits, misses, evictions, bytes copied, ring waits}
PK_EAPI int pk_expert_arena_ensure(void* h, const long long* keys, int n, void** out_ptrs, cudaStream_t stream, long long* stats) {
  return guarded([&] {
    auto* a = (pk::ExpertSlotArena*)h;
    a->ensure(keys, n, out_ptrs, stream);
    if (stats) {
      stats[0] = a->map().hits;
      stats[1] = a->map().misses;
      stats[2] = a->map().evictions;
      stats[3] = a->bytes_copied;
      stats[4] = a->ring().waits;
    }
  });
}

// Synchronous device-to-host copy of raw bytes (tests and tools that hold device addresses returned by this library).
PK_EAPI int pk_device_read(const void* device_ptr, void* host_out, unsigned long long bytes) {
  return guarded([&] {
    if (cudaMemcpy(host_out, device_ptr, (size_t)bytes, cudaMemcpyDeviceToHost) != cudaSuccess) throw std::runtime_error("pk_device_read: copy failed");
  });
}
