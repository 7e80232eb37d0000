// pocket_engine: command-line front end of the native engine, one process per rank.
//
// Flag surface and `key=value` result lines follow the reference's dsv4_cpp_engine for its
// Qwen path (cpp_engine/src/main.cpp:28-68, 407-746): --ckpt, --token-ids(-file),
// --max-new-tokens, --tp-world/--tp-rank, --device, --nccl-id-path (here: the rendezvous
// path for the peer-memory handles), --max-context, --prefill-chunk-tokens,
// --qwen-persistent-stdin, --qwen-attention-window/-sink-tokens, --dump-config, --inspect.
// Additions: --random-init SEED and --benchmark-27b run without a checkpoint.
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "control_plane.hpp"
#include "gguf_reader.hpp"
#include "json.hpp"
#include "openai_server.hpp"
#include <cmath>

#include "qwen_audit.hpp"
#include "qwen_config.hpp"
#include "qwen_engine.hpp"
#include "safetensors.hpp"
#include "tokenizer.hpp"
#include "weight_source.hpp"
#include "nccl_comm.hpp"

namespace {

struct Args {
  std::string ckpt, token_ids, token_ids_file, id_path = "/tmp/pocket_engine.rdv";
  int max_new_tokens = 16, tp_world = 1, tp_rank = 0, device = -1, max_context = 4096, prefill_chunk = 512;
  int window = 0, sink = 0;
  bool mtp = false, nccl_smoke = false, nccl_fallback = false;
  int mtp_tokens = 4;
  bool prefix_cache = true;
  int snapshot_interval = 4096, max_snapshots = 82;
  int persistent_decode = -1;
  int prefill_gemm = -1;
  std::string prompt_text, kv_cache_dtype = "bf16";
  long random_seed = -1;
  bool benchmark_27b = false, dump_config = false, inspect = false, persistent_stdin = false, no_graph = false;
  // serving
  bool serve = false, allow_shutdown = false, list_tensors = false;
  std::string host = "127.0.0.1", sidecar_python = "python", tokenizer = "chars", chat_format = "qwen", model_name = "pocketllm-b200";
  std::string fake_script, inspect_gguf, tokenizer_gguf, tokenizer_dir, tokenize_text, detokenize_ids;
  std::string weight_source, lookup, dsv4_config;
  int lookup_layer = -1, lookup_expert = -1;
  bool have_tokenize = false;
  bool fake_engine = false;
  int port = 8000;
  // checkpoint tools and smoke / bench modes
  std::string inspect_tensor, model_worker, worker_script = "Hello", worker_tokenizer_path;
  int worker_ranks = 1, worker_port = 29641;
  std::string qwen_dspark;   // directory of an external block drafter
  bool qwen_audit = false, smoke_forward = false;
  int smoke_layers = 4, resident_bench = 0;
};

void usage() {
  std::fprintf(stderr,
               "usage: pocket_engine --ckpt DIR | --benchmark-27b [--random-init SEED]\n"
               "  --token-ids 1,2,3 | --token-ids-file F   --max-new-tokens N\n"
               "  --tp-world N --tp-rank R --device D --nccl-id-path PATH\n"
               "  --max-context N --prefill-chunk-tokens N --no-cuda-graph\n"
               "  --qwen-attention-window N --qwen-attention-sink-tokens N\n"
               "  --qwen-mtp [--qwen-mtp-tokens K]   speculative decode with the checkpoint's multi-token predictor\n"
               "  --qwen-no-prefix-cache | --qwen-snapshot-interval N (4096, 0 = request boundaries only) --qwen-max-snapshots N (82)\n"
               "      exact prefix reuse across the requests of --qwen-persistent-stdin and --serve\n"
               "  --kv-cache-dtype bf16|fp8   --decode-kernel auto|persistent|per-projection\n"
               "  --prefill-gemm auto|fp8x2|fp8|shadow|umma   (many-row GEMM on the FP8 linears: native FP8 math with two or one\n"
               "                 E4M3 terms per activation, bf16 copies of the weights, or decode-to-bf16 in shared memory)\n"
               "  --prompt TEXT --tokenizer-gguf FILE   tokenise the prompt with the GGUF file's BPE vocabulary\n"
               "  --qwen-persistent-stdin | --dump-config | --inspect | --inspect-tensor NAME | --inspect-gguf FILE [--tensors]\n"
               "  --qwen-audit [--tp-world N] [--qwen-mtp]   check every tensor the engine reads (name, dtype, shape, shard cuts on the\n"
               "                 128-wide scale blocks) without a GPU; exit code 1 when something is wrong\n"
               "  --smoke-forward [--smoke-layers N]   random weights in the checkpoint's (or the benchmark) shape cut to N layers: one\n"
               "                 prefill and two decode steps\n"
               "  --generate-token   one new token (same as --max-new-tokens 1)   --resident-bench N   the request N times on the resident engine\n"
               "  --tokenizer-gguf FILE | --tokenizer-dir DIR (tokenizer.json)   --tokenize TEXT | --detokenize 1,2,3\n"
               "  --nccl-fallback   (with --tp-world > 1) join an NCCL communicator at start; after a peer wait times out the failed\n"
               "                 step is reported and later steps run their collectives through NCCL\n"
               "  --nccl-smoke --tp-world N --tp-rank R [--nccl-id-path PATH]   NCCL baseline path: all-reduce, broadcast, all-gather, top-1\n"
               "  --dsv4-config DIR|FILE.gguf [--tp-world N]   parse, validate and print a DeepSeek-V4 config\n"
               "  --weight-source DIR|FILE.gguf [--lookup NAME | --lookup-expert LAYER,EXPERT,w1|w2|w3]   tensor lookup by model name\n"
               "  --serve [--host H --port P --model-name N --tokenizer chars|hf:DIR|gguf:FILE --chat-format qwen|glm|minimax|dsv4\n"
               "           --sidecar-python EXE --fake-engine-script TEXT --allow-shutdown]\n"
               "  --serve --model-worker dsv4|gguf|qwen --ckpt PATH [--worker-tokenizer-path DIR] [--worker-ranks N]   serve a model family whose runtime is the\n"
               "                 Python one: this process is the HTTP / SSE front end, generation runs in a worker process\n"
               "                 (python -m pocketllm_b200.server.model_worker) on the GPU\n");
}

Args parse(int argc, char** argv) {
  Args a;
  auto need = [&](int& i) -> std::string {
    if (i + 1 >= argc) throw std::runtime_error(std::string("missing value for ") + argv[i]);
    return argv[++i];
  };
  for (int i = 1; i < argc; ++i) {
    const std::string f = argv[i];
    if (f == "--ckpt") a.ckpt = need(i);
    else if (f == "--model") need(i);  // accepted for compatibility; the checkpoint decides
    else if (f == "--token-ids") a.token_ids = need(i);
    else if (f == "--token-ids-file") a.token_ids_file = need(i);
    else if (f == "--max-new-tokens") a.max_new_tokens = std::stoi(need(i));
    else if (f == "--tp-world") a.tp_world = std::stoi(need(i));
    else if (f == "--tp-rank") a.tp_rank = std::stoi(need(i));
    else if (f == "--device") a.device = std::stoi(need(i));
    else if (f == "--nccl-id-path" || f == "--rendezvous-path") a.id_path = need(i);
    else if (f == "--max-context") a.max_context = std::stoi(need(i));
    else if (f == "--prefill-chunk-tokens") a.prefill_chunk = std::stoi(need(i));
    else if (f == "--qwen-attention-window") a.window = std::stoi(need(i));
    else if (f == "--qwen-attention-sink-tokens") a.sink = std::stoi(need(i));
    else if (f == "--nccl-smoke") a.nccl_smoke = true;
    else if (f == "--nccl-fallback") a.nccl_fallback = true;
    else if (f == "--qwen-mtp") a.mtp = true;
    else if (f == "--qwen-no-prefix-cache") a.prefix_cache = false;
    else if (f == "--qwen-snapshot-interval") a.snapshot_interval = std::stoi(need(i));
    else if (f == "--qwen-max-snapshots") a.max_snapshots = std::stoi(need(i));
    else if (f == "--kv-cache-dtype") {
      a.kv_cache_dtype = need(i);
      if (a.kv_cache_dtype == "fp16") a.kv_cache_dtype = "bf16";   // the reference's name for its 16-bit cache
      if (a.kv_cache_dtype != "bf16" && a.kv_cache_dtype != "fp8") throw std::runtime_error("--kv-cache-dtype must be bf16 (fp16) or fp8");
    }
    else if (f == "--prefill-gemm") {
      const std::string v = need(i);
      a.prefill_gemm = v == "umma" ? 0 : v == "shadow" ? 1 : v == "fp8x2" ? 2 : v == "fp8" ? 3 : -1;
    } else if (f == "--decode-kernel") {
      const std::string v = need(i);
      a.persistent_decode = v == "persistent" ? 1 : v == "per-projection" ? 0 : -1;
    }
    else if (f == "--prompt") a.prompt_text = need(i);
    else if (f == "--qwen-mtp-tokens") { a.mtp_tokens = std::stoi(need(i)); a.mtp = true; }
    else if (f == "--random-init") a.random_seed = std::stol(need(i));
    else if (f == "--benchmark-27b") a.benchmark_27b = true;
    else if (f == "--dump-config") a.dump_config = true;
    else if (f == "--inspect") a.inspect = true;
    else if (f == "--qwen-persistent-stdin") a.persistent_stdin = true;
    else if (f == "--no-cuda-graph") a.no_graph = true;
    else if (f == "--serve") a.serve = true;
    else if (f == "--host") a.host = need(i);
    else if (f == "--port") a.port = std::stoi(need(i));
    else if (f == "--model-name") a.model_name = need(i);
    else if (f == "--tokenizer") a.tokenizer = need(i);
    else if (f == "--chat-format") a.chat_format = need(i);
    else if (f == "--sidecar-python") a.sidecar_python = need(i);
    else if (f == "--fake-engine-script") { a.fake_script = need(i); a.fake_engine = true; }
    else if (f == "--allow-shutdown") a.allow_shutdown = true;
    else if (f == "--inspect-gguf") a.inspect_gguf = need(i);
    else if (f == "--tensors") a.list_tensors = true;
    else if (f == "--tokenizer-gguf") a.tokenizer_gguf = need(i);
    else if (f == "--tokenizer-dir") a.tokenizer_dir = need(i);
    else if (f == "--dsv4-config") a.dsv4_config = need(i);
    else if (f == "--weight-source") a.weight_source = need(i);
    else if (f == "--lookup") a.lookup = need(i);
    else if (f == "--lookup-expert") {
      const std::string v = need(i);
      const size_t c1 = v.find(','), c2 = v.find(',', c1 == std::string::npos ? 0 : c1 + 1);
      if (c1 == std::string::npos || c2 == std::string::npos) throw std::runtime_error("--lookup-expert wants LAYER,EXPERT,PART");
      a.lookup_layer = std::stoi(v.substr(0, c1));
      a.lookup_expert = std::stoi(v.substr(c1 + 1, c2 - c1 - 1));
      a.lookup = v.substr(c2 + 1);
    }
    else if (f == "--tokenize") { a.tokenize_text = need(i); a.have_tokenize = true; }
    else if (f == "--detokenize") a.detokenize_ids = need(i);
    else if (f == "--model-worker") a.model_worker = need(i);
    else if (f == "--worker-script") a.worker_script = need(i);
    else if (f == "--worker-ranks") a.worker_ranks = std::stoi(need(i));
    else if (f == "--worker-master-port") a.worker_port = std::stoi(need(i));
    else if (f == "--worker-tokenizer-path") a.worker_tokenizer_path = need(i);
    else if (f == "--inspect-tensor") a.inspect_tensor = need(i);
    else if (f == "--qwen-audit") a.qwen_audit = true;
    else if (f == "--smoke-forward") a.smoke_forward = true;
    else if (f == "--smoke-layers") a.smoke_layers = std::stoi(need(i));
    else if (f == "--generate-token") a.max_new_tokens = 1;
    else if (f == "--resident-bench") a.resident_bench = std::stoi(need(i));
    else if (f == "--use-persistent") a.persistent_decode = 1;   // the resident one-kernel-per-token decode path (the default where it applies)
    else if (f == "--qwen-mtp-adaptive") a.mtp = true;           // draft lengths always adapt (1, doubling after full accepts, halving after rejects)
    else if (f == "--python") a.sidecar_python = need(i);
    else if (f == "--sidecar") {}                                // --serve always runs the templating sidecar
    else if (f == "--forward-token" || f == "--position")
      throw std::runtime_error(f + ": the hybrid engine consumes positions in order (recurrent state); feed the tokens with --token-ids");
    else if (f == "--qwen-dspark") a.qwen_dspark = need(i);
    else if (f == "--help" || f == "-h") { usage(); std::exit(0); }
    else throw std::runtime_error("unknown flag " + f);
  }
  if (!a.qwen_dspark.empty()) {
    // the drafter's layers run in the Python runtime beside the engine: a served model gets both through a model worker
    if (!a.serve)
      throw std::runtime_error("--qwen-dspark: the external block drafter runs beside the engine in the Python runtime; serve it with "
                               "--serve --qwen-dspark DIR (model worker) or python -m pocketllm_b200.server.openai --model qwen --ckpt DIR --qwen-dspark DIR");
    if (a.model_worker.empty()) a.model_worker = "qwen";
    if (a.model_worker != "qwen") throw std::runtime_error("--qwen-dspark goes with the qwen model worker");
  }
  if (a.device < 0) a.device = a.tp_rank;
  return a;
}

std::vector<int> parse_ids(const std::string& text) {
  std::vector<int> out;
  std::string cur;
  for (char c : text + ",") {
    if (c == ',' || c == ' ' || c == '\n' || c == '\t') {
      if (!cur.empty()) out.push_back(std::stoi(cur));
      cur.clear();
    } else {
      cur.push_back(c);
    }
  }
  return out;
}

enum Op : int32_t { OP_GENERATE = 1, OP_RESET = 2, OP_SHUTDOWN = 3, OP_PREFILL = 4, OP_NEXT = 5, OP_SPEC = 6 };

int g_mtp_tokens = 4;   // draft length limit of speculative runs (--qwen-mtp-tokens)

// The Qwen engine behind the server. Greedy requests run the device sampler; with a temperature the
// logits of each step come back to the host sampler (single rank only: logits are vocabulary shards).
// With tensor parallelism rank 0 replays every step to the workers over the command channel. An engine built with the
// multi-token predictor serves greedy requests through speculative decode: tokens are produced a chunk at a time and
// handed out one by one (a request that stops inside a chunk simply leaves the rest unused; the next request resets).
class QwenTokenEngine : public pk::TokenEngine {
 public:
  QwenTokenEngine(pk::QwenEngine& e, pk::CmdChannel& chan, int world) : e_(e), chan_(chan), world_(world) {}
  int max_context() const override { return e_.options().max_context; }
  int prefill(const std::vector<int>& prompt, const pk::SamplerConfig& sc, uint64_t seed) override {
    sc_ = sc;
    rng_ = seed | 1;
    // logits come back to the host when the request samples or penalises (one rank: logits are vocabulary shards otherwise)
    host_sampling_ = (sc.temperature > 0.f || sc.has_penalties() || sc.logprobs >= 0) && world_ == 1;
    have_lp_ = false;
    produced_.clear();
    if (world_ > 1) {
      pk::CmdChannel::Message m;
      m.op = OP_PREFILL;
      m.payload.assign(prompt.begin(), prompt.end());
      chan_.broadcast(m);
    }
    buf_.clear();
    buf_pos_ = 0;
    try {
      const int first = e_.prefill_cached(prompt.data(), (int)prompt.size());   // reset + prefill when the cache is off
      return host_sampling_ ? resample(first) : first;
    } catch (const pk::CommTimeout& t) {
      throw pk::EngineStepFailed(t.what());   // HTTP 500; the status words are already cleared
    }
  }
  int next() override {
    try {
      return next_token();
    } catch (const pk::CommTimeout& t) {
      buf_.clear();
      buf_pos_ = 0;
      throw pk::EngineStepFailed(t.what());
    }
  }
  int next_token() {
    if (!host_sampling_ && e_.mtp_enabled()) {
      if (buf_pos_ < buf_.size()) return buf_[buf_pos_++];
      const int room = e_.options().max_context - e_.position() - 10;
      const int chunk = std::min(kSpecChunk, room);
      if (chunk >= 2) {
        if (world_ > 1) {
          pk::CmdChannel::Message m;
          m.op = OP_SPEC;
          m.payload = {chunk};
          chan_.broadcast(m);
        }
        buf_.assign((size_t)chunk, 0);
        pk::QwenSpecStats st;
        e_.spec_decode(chunk, g_mtp_tokens, buf_.data(), &st);
        spec_total_.rounds += st.rounds;
        spec_total_.proposed += st.proposed;
        spec_total_.accepted += st.accepted;
        spec_total_.rollbacks += st.rollbacks;
        buf_pos_ = 1;
        return buf_[0];
      }
    }
    if (world_ > 1) {
      pk::CmdChannel::Message m;
      m.op = OP_NEXT;
      chan_.broadcast(m);
    }
    if (host_sampling_) {
      int out = 0;
      e_.forward_rows(&last_, 1, &out);
      return resample(out);
    }
    int out = 0;
    e_.decode(1, &out, true);
    return out;
  }
  const pk::QwenSpecStats& spec_stats() const { return spec_total_; }
  bool last_logprobs(pk::TokenLogprobs* out) override {
    if (!host_sampling_ || !have_lp_) return false;      // several ranks: logits are vocabulary shards
    *out = lp_;
    return true;
  }

 private:
  int resample(int greedy) {
    logits_.resize((size_t)e_.vocab_local());
    e_.copy_logits(logits_.data(), 0);
    if (sc_.logprobs >= 0) raw_ = logits_;            // the model's distribution, before penalties
    pk::apply_penalties(logits_.data(), (int)logits_.size(), produced_, sc_);
    last_ = pk::sample_token(logits_.data(), (int)logits_.size(), sc_, rng_);
    if (sc_.logprobs >= 0) {
      pk::token_logprobs(raw_.data(), (int)raw_.size(), last_, sc_.logprobs, &lp_);
      have_lp_ = true;
    }
    produced_.push_back(last_);
    (void)greedy;
    return last_;
  }
  pk::QwenEngine& e_;
  pk::CmdChannel& chan_;
  int world_;
  pk::SamplerConfig sc_;
  uint64_t rng_ = 1;
  bool host_sampling_ = false;
  int last_ = 0;
  std::vector<float> logits_;
  std::vector<int> produced_;            // tokens of this request so far (for the penalties)
  std::vector<float> raw_;               // the step's logits before penalties (log-probability reports)
  pk::TokenLogprobs lp_;
  bool have_lp_ = false;
  static constexpr int kSpecChunk = 8;   // tokens produced per speculative call
  std::vector<int> buf_;                 // tokens of the current chunk not yet handed out
  size_t buf_pos_ = 0;
  pk::QwenSpecStats spec_total_;
};

std::vector<std::string> sidecar_command(const Args& a) {
  return {a.sidecar_python, "-m", "pocketllm_b200.server.cpp_sidecar", "--tokenizer", a.tokenizer, "--chat-format", a.chat_format};
}

int inspect_gguf(const Args& a) {
  pk::GgufFile f(a.inspect_gguf);
  std::map<std::string, std::pair<size_t, uint64_t>> by_type;
  uint64_t total = 0;
  for (const auto& t : f.tensors()) {
    auto& e = by_type[pk::ggml_type_name(t.type)];
    e.first += 1;
    e.second += t.nbytes;
    total += t.nbytes;
  }
  std::printf("gguf_version=%u architecture=%s alignment=%llu tensors=%zu metadata_keys=%zu tensor_bytes=%llu file_bytes=%llu\n", f.version(),
              f.architecture().c_str(), (unsigned long long)f.alignment(), f.tensors().size(), f.metadata().size(),
              (unsigned long long)total, (unsigned long long)f.file_size());
  for (const auto& kv : by_type)
    std::printf("type=%s tensors=%zu bytes=%llu\n", kv.first.c_str(), kv.second.first, (unsigned long long)kv.second.second);
  if (a.list_tensors) {
    for (const auto& t : f.tensors()) {
      std::printf("%s type=%s shape=[", t.name.c_str(), pk::ggml_type_name(t.type));
      for (size_t i = 0; i < t.dims.size(); ++i) std::printf(i ? ",%llu" : "%llu", (unsigned long long)t.dims[i]);
      std::printf("] offset=%llu bytes=%llu\n", (unsigned long long)t.offset, (unsigned long long)t.nbytes);
    }
  }
  return 0;
}

int serve_scripted(const Args& a) {
  auto eng = pk::make_scripted_engine(a.fake_script, a.max_context);
  pk::Sidecar sidecar(sidecar_command(a));
  pk::HttpServer http(a.host, a.port);
  std::printf("openai_server_listening host=%s port=%d engine=scripted\n", a.host.c_str(), http.port());
  std::fflush(stdout);
  pk::OpenAIServerOptions so;
  so.model_name = a.model_name;
  so.allow_shutdown = a.allow_shutdown;
  pk::run_openai_server(http, *eng, sidecar, so);
  return 0;
}

// The native front end in front of a Python model worker (DeepSeek-V4 runtime, GGUF runtimes).
int serve_worker(const Args& a) {
  std::vector<std::string> cmd = {a.sidecar_python};
  if (a.worker_ranks > 1) {
    // one worker rank per GPU: rank 0 inherits this pipe, the other ranks follow its requests
    for (const char* s : {"-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node"}) cmd.push_back(s);
    cmd.push_back(std::to_string(a.worker_ranks));
    for (const char* s : {"--master-addr", "127.0.0.1", "--master-port"}) cmd.push_back(s);
    cmd.push_back(std::to_string(a.worker_port));
  }
  for (const std::string& s : {std::string("-m"), std::string("pocketllm_b200.server.model_worker"), std::string("--model"), a.model_worker,
                               std::string("--max-context"), std::to_string(a.max_context)})
    cmd.push_back(s);
  if (!a.ckpt.empty()) { cmd.push_back("--ckpt"); cmd.push_back(a.ckpt); }
  if (!a.worker_tokenizer_path.empty()) { cmd.push_back("--tokenizer-path"); cmd.push_back(a.worker_tokenizer_path); }
  if (a.model_worker == "scripted") { cmd.push_back("--script"); cmd.push_back(a.worker_script); }
  if (!a.qwen_dspark.empty()) { cmd.push_back("--qwen-dspark"); cmd.push_back(a.qwen_dspark); }
  auto eng = pk::make_worker_engine(cmd);
  pk::Sidecar sidecar(sidecar_command(a));
  pk::HttpServer http(a.host, a.port);
  std::printf("openai_server_listening host=%s port=%d engine=worker model=%s\n", a.host.c_str(), http.port(), a.model_worker.c_str());
  std::fflush(stdout);
  pk::OpenAIServerOptions so;
  so.model_name = a.model_name;
  so.allow_shutdown = a.allow_shutdown;
  pk::run_openai_server(http, *eng, sidecar, so);
  return 0;
}

struct RunResult {
  std::vector<int> tokens;
  double prefill_s = 0, decode_s = 0;
  pk::QwenSpecStats spec;
};

// One request. `reuse` keeps the engine's state between requests and lets prefill_cached() skip the prefix it has
// already consumed (every rank takes the same decision: it depends on the token sequences only).
RunResult generate(pk::QwenEngine& eng, const std::vector<int>& prompt, int max_new, bool reuse = false) {
  RunResult r;
  int first;
  if (reuse) {
    first = eng.prefill_cached(prompt.data(), (int)prompt.size());
  } else {
    eng.reset();
    first = eng.prefill(prompt.data(), (int)prompt.size());
  }
  r.tokens.push_back(first);
  r.prefill_s = eng.timings().prefill_ms / 1e3;
  if (max_new > 1) {
    std::vector<int> rest(max_new - 1);
    if (eng.mtp_enabled()) eng.spec_decode(max_new - 1, g_mtp_tokens, rest.data(), &r.spec);
    else eng.decode(max_new - 1, rest.data(), false);
    r.tokens.insert(r.tokens.end(), rest.begin(), rest.end());
    r.decode_s = eng.timings().decode_ms / 1e3;
  }
  return r;
}

void print_result(const char* tag, const Args& a, const pk::QwenEngine& eng, size_t prompt_len, const RunResult& r) {
  std::printf("%s=1 tp_world=%d tp_rank=%d prompt_tokens=%zu generated_tokens=%zu prefill_seconds=%.6f "
              "prefill_tokens_per_s=%.3f decode_seconds=%.6f decode_tokens_per_s=%.3f weight_bytes=%zu generated_token_ids=",
              tag, a.tp_world, a.tp_rank, prompt_len, r.tokens.size(), r.prefill_s,
              r.prefill_s > 0 ? prompt_len / r.prefill_s : 0.0, r.decode_s,
              r.decode_s > 0 ? (r.tokens.size() - 1) / r.decode_s : 0.0, eng.weight_bytes());
  for (size_t i = 0; i < r.tokens.size(); ++i) std::printf(i ? ",%d" : "%d", r.tokens[i]);
  if (eng.mtp_enabled())
    std::printf(" mtp_rounds=%lld mtp_proposed=%lld mtp_accepted=%lld mtp_rollbacks=%lld mtp_replay_tokens=%lld mtp_plain_steps=%lld",
                r.spec.rounds, r.spec.proposed, r.spec.accepted, r.spec.rollbacks, r.spec.replay_tokens, r.spec.plain_steps);
  if (eng.options().prefix_cache && std::strcmp(tag, "qwen_runtime") != 0) {
    const pk::QwenPrefixStats& ps = eng.prefix_stats();
    std::printf(" prefix_reused_tokens=%d prefix_computed_tokens=%d prefix_matched_tokens=%d prefix_resume=%s prefix_snapshots=%d "
                "prefix_snapshot_bytes=%llu prefix_hits=%lld prefix_misses=%lld",
                ps.reused_tokens, ps.computed_tokens, ps.matched_tokens, ps.resume_source, ps.snapshots, ps.snapshot_bytes, ps.hits, ps.misses);
  }
  std::printf("\n");
  std::fflush(stdout);
}

void print_view(const pk::TensorView& v) {
  if (!v.found) {
    std::printf("tensor=%s found=0\n", v.name.c_str());
    return;
  }
  unsigned long long sum = 0;
  for (uint64_t i = 0; i < v.nbytes; ++i) sum += v.data[i];
  std::printf("tensor=%s found=1 stored=%s dtype=%s shape=[", v.name.c_str(), v.stored_name.c_str(), v.dtype.c_str());
  for (size_t i = 0; i < v.shape.size(); ++i) std::printf(i ? ",%lld" : "%lld", (long long)v.shape[i]);
  std::printf("] bytes=%llu byte_sum=%llu\n", (unsigned long long)v.nbytes, sum);
}

int weight_source_tool(const Args& a) {
  auto src = pk::open_weight_source(a.weight_source);
  std::printf("format=%s\n", src->format() == pk::WeightSource::Format::Gguf ? "gguf" : "safetensors");
  if (a.lookup_layer >= 0) print_view(src->expert(a.lookup_layer, a.lookup_expert, a.lookup));
  else if (!a.lookup.empty()) print_view(src->get(a.lookup));
  else
    for (const std::string& n : src->names()) print_view(src->get(n));
  return 0;
}

int dsv4_config_tool(const Args& a) {
  pk::Dsv4Config cfg;
  if (pk::is_gguf_path(a.dsv4_config)) {
    pk::GgufFile f(a.dsv4_config);
    cfg = pk::Dsv4Config::from_gguf(f);
  } else {
    const bool is_file = a.dsv4_config.size() > 5 && a.dsv4_config.compare(a.dsv4_config.size() - 5, 5, ".json") == 0;
    cfg = pk::Dsv4Config::from_file(is_file ? a.dsv4_config : a.dsv4_config + "/config.json");
  }
  cfg.validate(a.tp_world);
  std::printf("%s\n", cfg.to_json().dump().c_str());
  return 0;
}

// Sum, broadcast, gather and global top-1 through the NCCL baseline path; every rank prints its verdict.
int nccl_smoke(const Args& a) {
  if (!pk::NcclComm::available()) {
    std::printf("nccl_smoke=1 available=0\n");
    return 0;
  }
  pk::NcclComm comm(a.id_path, a.tp_rank, a.tp_world, a.device);
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  const int n = 4096, W = a.tp_world, R = a.tp_rank;
  std::vector<float> host(n, (float)(R + 1));
  float* buf = nullptr;
  float* all = nullptr;
  int* tok = nullptr;
  cudaMalloc((void**)&buf, n * sizeof(float));
  cudaMalloc((void**)&all, (size_t)n * W * sizeof(float));
  cudaMalloc((void**)&tok, sizeof(int));
  cudaMemcpy(buf, host.data(), n * sizeof(float), cudaMemcpyHostToDevice);
  comm.all_gather(buf, all, n, pk::NcclComm::Dtype::F32, stream);
  comm.all_reduce_sum(buf, n, pk::NcclComm::Dtype::F32, stream);
  int t = R == 0 ? 4242 : -1;
  cudaMemcpy(tok, &t, sizeof(int), cudaMemcpyHostToDevice);
  comm.broadcast(tok, 1, pk::NcclComm::Dtype::I32, 0, stream);
  cudaStreamSynchronize(stream);
  std::vector<float> gathered((size_t)n * W);
  cudaMemcpy(host.data(), buf, n * sizeof(float), cudaMemcpyDeviceToHost);
  cudaMemcpy(gathered.data(), all, gathered.size() * sizeof(float), cudaMemcpyDeviceToHost);
  cudaMemcpy(&t, tok, sizeof(int), cudaMemcpyDeviceToHost);
  const float want = (float)(W * (W + 1) / 2);
  bool ok = t == 4242;
  for (int i = 0; i < n; ++i) ok = ok && host[i] == want;
  for (int r = 0; r < W; ++r) ok = ok && gathered[(size_t)r * n] == (float)(r + 1) && gathered[(size_t)r * n + n - 1] == (float)(r + 1);
  // the highest rank holds the best logit; equal logits on the others resolve to the lowest token
  float best = 0.f;
  const int top = comm.global_top1(R == W - 1 ? 9.f : 1.f, 1000 + R, stream, &best);
  ok = ok && top == 1000 + W - 1 && best == 9.f;
  std::printf("nccl_smoke=1 available=1 tp_world=%d tp_rank=%d ok=%d sum=%.1f broadcast=%d top1=%d\n", W, R, ok ? 1 : 0, host[0], t, top);
  cudaFree(buf);
  cudaFree(all);
  cudaFree(tok);
  cudaStreamDestroy(stream);
  return ok ? 0 : 1;
}

pk::BpeTokenizer load_tokenizer(const Args& a) {
  if (!a.tokenizer_dir.empty()) return pk::BpeTokenizer::from_hf_dir(a.tokenizer_dir);
  if (a.tokenizer_gguf.empty()) throw std::runtime_error("give --tokenizer-gguf FILE or --tokenizer-dir DIR for the vocabulary");
  pk::GgufFile f(a.tokenizer_gguf);
  return pk::BpeTokenizer::from_gguf(f);
}

int tokenizer_tool(const Args& a) {
  const pk::BpeTokenizer tok = load_tokenizer(a);
  if (a.have_tokenize) {
    const std::vector<int> ids = tok.encode(a.tokenize_text);
    std::printf("token_ids=");
    for (size_t i = 0; i < ids.size(); ++i) std::printf(i ? ",%d" : "%d", ids[i]);
    std::printf("\n");
  }
  if (!a.detokenize_ids.empty()) std::printf("text=%s\n", tok.decode(parse_ids(a.detokenize_ids)).c_str());
  return 0;
}

// First values of a tensor as floats (the dtypes checkpoints use).
double element_as_double(const pk::StTensor& t, int64_t i) {
  const uint8_t* p = t.data;
  switch (t.dtype) {
    case pk::StDtype::F32: { float v; std::memcpy(&v, p + 4 * i, 4); return v; }
    case pk::StDtype::BF16: { uint16_t h; std::memcpy(&h, p + 2 * i, 2); const uint32_t u = (uint32_t)h << 16; float v; std::memcpy(&v, &u, 4); return v; }
    case pk::StDtype::F16: {
      uint16_t h; std::memcpy(&h, p + 2 * i, 2);
      const int sgn = h >> 15, e = (h >> 10) & 31, m = h & 1023;
      const double mag = e == 0 ? std::ldexp((double)m, -24) : e == 31 ? (m ? NAN : INFINITY) : std::ldexp((double)(m + 1024), e - 25);
      return sgn ? -mag : mag;
    }
    case pk::StDtype::F8_E4M3: {
      const uint8_t b = p[i];
      const int sgn = b >> 7, e = (b >> 3) & 15, m = b & 7;
      const double mag = e == 0 ? std::ldexp((double)m, -9) : (e == 15 && m == 7) ? NAN : std::ldexp((double)(m + 8), e - 10);
      return sgn ? -mag : mag;
    }
    case pk::StDtype::F8_E8M0: return std::ldexp(1.0, (int)p[i] - 127);
    case pk::StDtype::I8: return (int8_t)p[i];
    case pk::StDtype::U8: return p[i];
    case pk::StDtype::I32: { int32_t v; std::memcpy(&v, p + 4 * i, 4); return v; }
    case pk::StDtype::I64: { int64_t v; std::memcpy(&v, p + 8 * i, 8); return (double)v; }
    default: return NAN;
  }
}

int inspect_tensor(const Args& a) {
  pk::SafetensorsModel st(a.ckpt);
  const pk::StTensor* t = st.find(a.inspect_tensor);
  if (t == nullptr) {
    std::printf("tensor=%s found=0\n", a.inspect_tensor.c_str());
    return 1;
  }
  std::printf("tensor=%s found=1 dtype=%s shape=[", t->name.c_str(), pk::st_dtype_name(t->dtype));
  for (size_t i = 0; i < t->shape.size(); ++i) std::printf(i ? ",%lld" : "%lld", (long long)t->shape[i]);
  std::printf("] bytes=%zu first=[", t->nbytes);
  const int64_t n = std::min<int64_t>(8, t->numel());
  for (int64_t i = 0; i < n; ++i) std::printf(i ? ",%.9g" : "%.9g", element_as_double(*t, i));
  double sum = 0.0, amax = 0.0;
  for (int64_t i = 0; i < t->numel(); ++i) {
    const double v = element_as_double(*t, i);
    sum += v;
    amax = std::max(amax, std::fabs(v));
  }
  std::printf("] sum=%.9g abs_max=%.9g\n", sum, amax);
  return 0;
}

int qwen_audit(const Args& a) {
  pk::SafetensorsModel st(a.ckpt);
  const pk::QwenConfig cfg = pk::QwenConfig::from_file(a.ckpt + "/config.json");
  bool config_ok = true;
  try {
    cfg.validate(a.tp_world);
  } catch (const std::exception& e) {
    std::printf("qwen_audit_problem=config %s\n", e.what());
    config_ok = false;
  }
  const pk::QwenAuditReport rep = pk::audit_qwen_checkpoint(st, cfg, a.tp_world, a.mtp);
  for (const std::string& p : rep.problems) std::printf("qwen_audit_problem=%s\n", p.c_str());
  for (const std::string& u : rep.unused) std::printf("qwen_audit_unused=%s\n", u.c_str());
  const bool ok = rep.ok() && config_ok;
  std::printf("qwen_audit=1 ok=%d tp_world=%d layers=%d expected_tensors=%d fp8_linears=%d problems=%zu unused_tensors=%zu expected_bytes=%llu files=%zu\n",
              ok ? 1 : 0, a.tp_world, cfg.num_layers, rep.expected, rep.fp8_linears, rep.problems.size() + (config_ok ? 0 : 1), rep.unused.size(),
              (unsigned long long)rep.expected_bytes, st.num_files());
  return ok ? 0 : 1;
}

int run(const Args& a) {
  if ((!a.tokenizer_gguf.empty() || !a.tokenizer_dir.empty()) && (a.have_tokenize || !a.detokenize_ids.empty())) return tokenizer_tool(a);
  if (!a.inspect_gguf.empty()) return inspect_gguf(a);
  if (a.nccl_smoke) return nccl_smoke(a);
  if (!a.dsv4_config.empty()) return dsv4_config_tool(a);
  if (!a.weight_source.empty()) return weight_source_tool(a);
  if (a.serve && a.fake_engine) return serve_scripted(a);
  if (a.serve && !a.model_worker.empty()) return serve_worker(a);
  if (!a.inspect_tensor.empty()) return inspect_tensor(a);
  if (a.qwen_audit) return qwen_audit(a);
  if (a.inspect) {
    pk::SafetensorsModel st(a.ckpt);
    for (const auto& n : st.names()) {
      const pk::StTensor& t = st.get(n);
      std::printf("%s dtype=%s shape=[", n.c_str(), pk::st_dtype_name(t.dtype));
      for (size_t i = 0; i < t.shape.size(); ++i) std::printf(i ? ",%lld" : "%lld", (long long)t.shape[i]);
      std::printf("] bytes=%zu\n", t.nbytes);
    }
    return 0;
  }
  pk::QwenConfig cfg = (a.benchmark_27b || (a.smoke_forward && a.ckpt.empty())) ? pk::QwenConfig::benchmark_27b() : pk::QwenConfig::from_file(a.ckpt + "/config.json");
  if (a.smoke_forward) {
    // the shape of the model, the first N layers only, random weights: seconds instead of a full load
    const int n = std::max(1, std::min(a.smoke_layers, cfg.num_layers));
    cfg.num_layers = n;
    cfg.layer_is_full.resize((size_t)n);
    cfg.mtp_num_hidden_layers = 0;
  }
  if (a.dump_config) {
    std::printf("%s\n", cfg.to_json().c_str());
    return 0;
  }
  pk::QwenEngineOptions opt;
  opt.tp_rank = a.tp_rank;
  opt.tp_world = a.tp_world;
  opt.device = a.device;
  opt.max_context = a.max_context;
  opt.prefill_chunk = a.prefill_chunk;
  opt.use_cuda_graph = !a.no_graph;
  opt.attention_window = a.window;
  opt.attention_sink = a.sink;
  opt.mtp = a.mtp;
  opt.kv_fp8 = a.kv_cache_dtype == "fp8";
  opt.prefix_cache = a.prefix_cache;
  opt.snapshot_interval = a.snapshot_interval;
  opt.max_snapshots = a.max_snapshots;
  opt.persistent_decode = a.persistent_decode;
  opt.prefill_gemm = a.prefill_gemm;
  g_mtp_tokens = a.mtp_tokens;
  pk::QwenEngine eng(cfg, opt);
  if (a.random_seed >= 0 || a.benchmark_27b || a.smoke_forward) eng.init_random((uint64_t)std::max(0L, a.random_seed), 0.02f);
  else eng.load_safetensors(a.ckpt);

  std::vector<void*> opened;
  if (a.tp_world > 1) {
    // Exchange the arenas' IPC handles through files, then map the peers.
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, eng.comm_arena()) != cudaSuccess) throw std::runtime_error("cudaIpcGetMemHandle failed");
    std::vector<uint8_t> blob(sizeof h);
    std::memcpy(blob.data(), &h, sizeof h);
    auto all = pk::file_rendezvous(a.id_path, a.tp_rank, a.tp_world, blob);
    std::vector<void*> arenas(a.tp_world, nullptr);
    for (int r = 0; r < a.tp_world; ++r) {
      if (r == a.tp_rank) continue;
      cudaIpcMemHandle_t ph;
      std::memcpy(&ph, all[r].data(), sizeof ph);
      if (cudaIpcOpenMemHandle(&arenas[r], ph, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
        throw std::runtime_error("cudaIpcOpenMemHandle failed for rank " + std::to_string(r));
      opened.push_back(arenas[r]);
    }
    eng.set_peer_arenas(arenas.data());
    // joined now, while every rank is known to be up; used only after a bounded peer wait has run out
    if (a.nccl_fallback) eng.enable_nccl_fallback(a.id_path + ".nccl");
  }
  pk::CmdChannel chan(a.id_path + ".cmdsock", a.tp_rank, a.tp_world);
  if (a.tp_world > 1) pk::file_rendezvous_cleanup(a.id_path, a.tp_rank);

  int rc = 0;
  if (a.serve) {
    if (a.tp_rank == 0) {
      QwenTokenEngine te(eng, chan, a.tp_world);
      pk::Sidecar sidecar(sidecar_command(a));
      pk::HttpServer http(a.host, a.port);
      std::printf("openai_server_listening host=%s port=%d engine=qwen tp_world=%d\n", a.host.c_str(), http.port(), a.tp_world);
      std::fflush(stdout);
      pk::OpenAIServerOptions so;
      so.model_name = a.model_name;
      so.allow_shutdown = a.allow_shutdown;
      pk::run_openai_server(http, te, sidecar, so);
      if (eng.mtp_enabled())
        std::printf("serve_mtp_rounds=%lld serve_mtp_proposed=%lld serve_mtp_accepted=%lld serve_mtp_rollbacks=%lld\n", te.spec_stats().rounds,
                    te.spec_stats().proposed, te.spec_stats().accepted, te.spec_stats().rollbacks);
      pk::CmdChannel::Message bye;
      bye.op = OP_SHUTDOWN;
      chan.broadcast(bye);
    } else {
      pk::CmdChannel::Message m;
      while (chan.receive(m)) {
        if (m.op == OP_SHUTDOWN) break;
        try {
          if (m.op == OP_PREFILL) {
            std::vector<int> prompt(m.payload.begin(), m.payload.end());
            eng.prefill_cached(prompt.data(), (int)prompt.size());
          } else if (m.op == OP_NEXT) {
            int out = 0;
            eng.decode(1, &out, true);
          } else if (m.op == OP_SPEC && !m.payload.empty()) {
            eng.spec_decode(m.payload[0], g_mtp_tokens, nullptr, nullptr);
          }
        } catch (const std::exception& e) {
          std::fprintf(stderr, "worker %d: %s\n", a.tp_rank, e.what());
        }
      }
    }
  } else if (a.persistent_stdin) {
    // Rank 0 reads "<max_new_tokens> tok0 tok1 ..." lines ("reset" / "quit" also accepted) and
    // replays them to the workers; every rank runs the same generate.
    if (a.tp_rank == 0) {
      std::string line;
      while (std::getline(std::cin, line)) {
        if (line == "quit" || line == "shutdown") break;
        pk::CmdChannel::Message m;
        if (line == "reset") {
          m.op = OP_RESET;
          chan.broadcast(m);
          eng.clear_prefix_cache();
          eng.reset();
          std::printf("qwen_persistent_reset=1\n");
          std::fflush(stdout);
          continue;
        }
        std::vector<int> nums = parse_ids(line);
        if (nums.size() < 2) {
          std::printf("qwen_persistent_error=1 message=expected_max_new_tokens_then_token_ids\n");
          std::fflush(stdout);
          continue;
        }
        m.op = OP_GENERATE;
        m.payload.assign(nums.begin(), nums.end());
        chan.broadcast(m);
        std::vector<int> prompt(nums.begin() + 1, nums.end());
        try {
          RunResult r = generate(eng, prompt, nums[0], true);
          print_result("qwen_persistent_result", a, eng, prompt.size(), r);
        } catch (const std::exception& e) {
          std::printf("qwen_persistent_error=1 message=%s\n", e.what());
          std::fflush(stdout);
        }
      }
      pk::CmdChannel::Message bye;
      bye.op = OP_SHUTDOWN;
      chan.broadcast(bye);
    } else {
      pk::CmdChannel::Message m;
      while (chan.receive(m)) {  // blocks in recv(): an idle worker uses no GPU and no CPU
        if (m.op == OP_SHUTDOWN) break;
        if (m.op == OP_RESET) {
          eng.clear_prefix_cache();
          eng.reset();
          continue;
        }
        if (m.op == OP_GENERATE && m.payload.size() >= 2) {
          std::vector<int> prompt(m.payload.begin() + 1, m.payload.end());
          try {
            generate(eng, prompt, m.payload[0], true);
          } catch (const std::exception& e) {
            std::fprintf(stderr, "worker %d: %s\n", a.tp_rank, e.what());
          }
        }
      }
    }
  } else {
    std::vector<int> prompt;
    if (!a.token_ids_file.empty()) {
      std::ifstream in(a.token_ids_file);
      std::stringstream ss;
      ss << in.rdbuf();
      prompt = parse_ids(ss.str());
    } else if (!a.prompt_text.empty()) {
      prompt = load_tokenizer(a).encode(a.prompt_text);
    } else {
      prompt = parse_ids(a.token_ids);
    }
    if (prompt.empty() && a.smoke_forward) prompt = {1, 2, 3, 4};
    if (prompt.empty()) throw std::runtime_error("no prompt: give --token-ids, --token-ids-file or --prompt");
    if (a.smoke_forward) {
      RunResult r = generate(eng, prompt, 3);
      const bool fine = r.tokens.size() == 3 && eng.comm_status() == 0;
      std::printf("smoke_forward=1 ok=%d layers=%d prompt_tokens=%zu generated_token_ids=%d,%d,%d\n", fine ? 1 : 0, cfg.num_layers, prompt.size(),
                  r.tokens[0], r.tokens.size() > 1 ? r.tokens[1] : -1, r.tokens.size() > 2 ? r.tokens[2] : -1);
      for (void* p : opened) cudaIpcCloseMemHandle(p);
      return fine ? 0 : 1;
    }
    if (a.resident_bench > 0) {
      // the same request again and again on the resident engine (weights, caches and graphs stay): one line per run
      double pf = 0, dc = 0;
      for (int it = 0; it < a.resident_bench; ++it) {
        RunResult rr = generate(eng, prompt, a.max_new_tokens);
        print_result("qwen_resident_run", a, eng, prompt.size(), rr);
        pf += rr.prefill_s > 0 ? prompt.size() / rr.prefill_s : 0.0;
        dc += rr.decode_s > 0 ? (rr.tokens.size() - 1) / rr.decode_s : 0.0;
      }
      std::printf("qwen_resident_bench=1 runs=%d prefill_tokens_per_s_mean=%.3f decode_tokens_per_s_mean=%.3f comm_status=%u\n", a.resident_bench,
                  pf / a.resident_bench, dc / a.resident_bench, eng.comm_status());
      for (void* p : opened) cudaIpcCloseMemHandle(p);
      return eng.comm_status() == 0 ? 0 : 3;
    }
    RunResult r = generate(eng, prompt, a.max_new_tokens);
    if (eng.comm_status() != 0) {
      std::printf("qwen_comm_status=%u\n", eng.comm_status());
      rc = 3;
    }
    print_result("qwen_runtime", a, eng, prompt.size(), r);
  }
  for (void* p : opened) cudaIpcCloseMemHandle(p);
  return rc;
}

}  // namespace

int main(int argc, char** argv) {
  try {
    return run(parse(argc, argv));
  } catch (const std::exception& e) {
    std::fprintf(stderr, "pocket_engine: %s\n", e.what());
    return 1;
  }
}
