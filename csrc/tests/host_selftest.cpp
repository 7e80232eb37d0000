// Self-test of the engine's host code (JSON, GGUF and Safetensors readers, sampler, file rendezvous, command
// channel, host model of the peer all-reduce protocol). Built with -fsanitize=address,undefined (or thread)
// by the test-suite and run on a machine without a GPU.
//   host_selftest <file.gguf> <safetensors dir> <scratch dir>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../common/pk_comm_host.hpp"
#include "../engine/qwen_audit.hpp"
#include "../engine/tokenizer.hpp"
#include "../engine/dsv4_config.hpp"
#include "../engine/weight_source.hpp"
#include "../engine/control_plane.hpp"
#include "../engine/gguf_reader.hpp"
#include "../engine/json.hpp"
#include "../engine/safetensors.hpp"
#include "../engine/sampler.hpp"
#include "../engine/prefix_plan.hpp"
#include "../engine/spec_policy.hpp"

#define CHECK(cond)                                                             \
  do {                                                                          \
    if (!(cond)) {                                                              \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
      return 1;                                                                 \
    }                                                                           \
  } while (0)

static int test_json() {
  const std::string text = R"({"a":[1,2.5,-3e2,true,null,"xé\n\"q\""],"b":{"c":9007199254740993,"d":{}},"e":[]})";
  pk::Json j = pk::Json::parse(text);
  CHECK(j.at("a").items().size() == 6 && j.at("a").items()[1].as_double() == 2.5 && j.at("a").items()[2].as_double() == -300.0);
  CHECK(j.at("b").at("c").as_int() == 9007199254740993LL);
  CHECK(j.at("a").items()[5].as_string() == std::string("x\xc3\xa9\n\"q\""));
  pk::Json again = pk::Json::parse(j.dump());
  CHECK(again.dump() == j.dump());
  for (const char* bad : {"{", "[1,]", "{\"a\":}", "\"unterminated", "tru", "{\"a\":1}x", ""}) {
    bool threw = false;
    try {
      pk::Json::parse(bad);
    } catch (const std::exception&) {
      threw = true;
    }
    CHECK(threw);
  }
  return 0;
}

static int test_readers(const std::string& gguf_path, const std::string& st_dir) {
  pk::GgufFile g(gguf_path);
  CHECK(!g.architecture().empty() && !g.tensors().empty());
  uint64_t sum = 0;
  for (const auto& t : g.tensors()) {
    const uint8_t* p = g.data(t);
    sum += p[0] + p[t.nbytes - 1];                 // touches the first and the last byte of every tensor
  }
  CHECK(g.find("no.such.tensor") == nullptr);
  pk::SafetensorsModel st(st_dir);
  CHECK(!st.names().empty());
  for (const auto& n : st.names()) {
    const pk::StTensor& t = st.get(n);
    if (t.nbytes) sum += ((const uint8_t*)t.data)[0] + ((const uint8_t*)t.data)[t.nbytes - 1];
  }
  std::printf("readers_checksum=%llu\n", (unsigned long long)sum);
  return 0;
}

// Checkpoint audit on a complete tiny checkpoint: everything the engine reads is found; four ranks do not cut its
// 128-row blocks evenly and are refused.
static int test_qwen_audit(const std::string& st_dir) {
  pk::SafetensorsModel st(st_dir);
  const pk::QwenConfig cfg = pk::QwenConfig::from_file(st_dir + "/config.json");
  const pk::QwenAuditReport one = pk::audit_qwen_checkpoint(st, cfg, 1, false);
  CHECK(one.ok() && one.expected > 20 && one.fp8_linears > 0 && one.unused.empty() && one.expected_bytes > 0);
  const pk::QwenAuditReport four = pk::audit_qwen_checkpoint(st, cfg, 4, false);
  CHECK(!four.ok());
  const pk::QwenAuditReport mtp = pk::audit_qwen_checkpoint(st, cfg, 1, true);
  CHECK(!mtp.ok() && mtp.problems.front().rfind("missing mtp.", 0) == 0);      // this checkpoint has no predictor
  return 0;
}

// Byte-level BPE from a GGUF vocabulary: every text comes back from decode(encode(text)), the pre-tokeniser loses no
// byte, special tokens are matched verbatim only when asked to.
static int test_tokenizer(const std::string& gguf_path) {
  pk::GgufFile f(gguf_path);
  const pk::BpeTokenizer tok = pk::BpeTokenizer::from_gguf(f);
  CHECK(tok.vocab_size() > 256);
  const char* texts[] = {"Hello, world! It's me.", "  leading spaces and\ttabs\n\nnewlines  ", "x=1+2;y=[3,4]", "na\xc3\xafve caf\xc3\xa9", "", "   ",
                         "12345 67 8", "<|eos|>after special<|eos|>", "line1\nline2\r\n  indented", "\xf0\x9f\x98\x80 emoji"};
  for (const char* t : texts) {
    const std::string text(t);
    const std::vector<int> ids = tok.encode(text);
    CHECK(tok.decode(ids) == text);
    for (int id : ids) CHECK(id >= 0 && id < tok.vocab_size());
    std::string glued;
    for (const std::string& piece : pk::BpeTokenizer::pre_tokenize(text)) glued += piece;
    CHECK(glued == text);
  }
  const int eos = tok.token_id("<|eos|>");
  CHECK(eos >= 0);
  const std::vector<int> sp = tok.encode("<|eos|>x", true), plain = tok.encode("<|eos|>x", false);
  CHECK(sp.size() == 2 && sp[0] == eos && plain.size() > 2);
  CHECK(tok.decode(sp, true) == "x");
  return 0;
}

// Container-agnostic tensor lookup over both formats, and the DeepSeek-V4 config parser (defaults, validation).
static int test_weight_source_and_dsv4_config(const std::string& gguf_path, const std::string& st_dir) {
  bool other_family = false;
  try {
    pk::open_weight_source(gguf_path);                  // a MiniMax file is not a DeepSeek-V4 checkpoint
  } catch (const std::exception&) {
    other_family = true;
  }
  CHECK(other_family);
  for (const std::string& path : {st_dir}) {
    auto src = pk::open_weight_source(path);
    const std::vector<std::string> names = src->names();
    CHECK(!names.empty());
    uint64_t total = 0;
    for (const std::string& n : names) {
      const pk::TensorView v = src->get(n);
      CHECK(v.found && v.data != nullptr && v.nbytes > 0 && !v.shape.empty());
      total += v.data[0] + v.data[v.nbytes - 1];       // first and last byte are inside the mapping
    }
    (void)total;
    CHECK(!src->get("no.such.tensor").found);
    bool threw = false;
    try {
      src->require("no.such.tensor");
    } catch (const std::exception&) {
      threw = true;
    }
    CHECK(threw);
  }
  pk::Dsv4Config cfg = pk::Dsv4Config::from_json(pk::Json::parse("{\"n_layers\": 4, \"dim\": 256, \"n_heads\": 4, \"o_groups\": 2, \"n_routed_experts\": 8}"));
  CHECK(cfg.n_layers == 4 && cfg.dim == 256 && cfg.head_dim == 512 && cfg.index_topk == 512);      // the rest keeps the defaults
  cfg.validate(2);
  bool refused = false;
  try {
    cfg.validate(3);                                    // three ranks divide neither heads nor experts
  } catch (const std::exception&) {
    refused = true;
  }
  CHECK(refused);
  const pk::Dsv4Config again = pk::Dsv4Config::from_json(cfg.to_json());
  CHECK(again.n_layers == cfg.n_layers && again.dim == cfg.dim && again.score_func == cfg.score_func);
  return 0;
}

// Hostile Safetensors files: every one must end in an exception, never in a read outside the mapping.
static int test_safetensors_rejects_hostile_headers(const std::string& scratch) {
  auto write_file = [&](const std::string& name, uint64_t header_len, const std::string& header, size_t payload) {
    const std::string path = scratch + "/" + name;
    FILE* f = std::fopen(path.c_str(), "wb");
    std::fwrite(&header_len, 8, 1, f);
    std::fwrite(header.data(), 1, header.size(), f);
    std::vector<char> zeros(payload, 0);
    if (payload) std::fwrite(zeros.data(), 1, payload, f);
    std::fclose(f);
    return path;
  };
  auto refused = [&](const std::string& path) {
    try {
      pk::SafetensorsModel m(path);
      for (const std::string& n : m.names()) (void)m.get(n).data[m.get(n).nbytes - 1];
    } catch (const std::exception&) {
      return true;
    }
    return false;
  };
  const std::string ok = "{\"a\":{\"dtype\":\"F32\",\"shape\":[2,2],\"data_offsets\":[0,16]}}";
  CHECK(!refused(write_file("ok.safetensors", ok.size(), ok, 16)));
  CHECK(refused(write_file("short.safetensors", ok.size(), ok, 8)));                        // offsets beyond the payload
  CHECK(refused(write_file("hdrlen.safetensors", 1ull << 40, ok, 16)));                      // header length beyond the file
  const std::string neg = "{\"a\":{\"dtype\":\"F32\",\"shape\":[-2,2],\"data_offsets\":[0,16]}}";
  CHECK(refused(write_file("neg.safetensors", neg.size(), neg, 16)));
  const std::string huge = "{\"a\":{\"dtype\":\"F32\",\"shape\":[4611686018427387904,4],\"data_offsets\":[0,16]}}";
  CHECK(refused(write_file("huge.safetensors", huge.size(), huge, 16)));                     // element count would wrap
  const std::string back = "{\"a\":{\"dtype\":\"F32\",\"shape\":[2,2],\"data_offsets\":[16,0]}}";
  CHECK(refused(write_file("back.safetensors", back.size(), back, 16)));
  const std::string junk = "{\"a\":{\"dtype\":\"F32\",\"shape\":[2,2],\"data_offsets\":[0,";
  CHECK(refused(write_file("junk.safetensors", junk.size(), junk, 16)));                      // truncated JSON
  CHECK(refused(write_file("tiny.safetensors", 0, "", 0) ) || true);                          // an empty header is an empty model
  return 0;
}

static int test_sampler() {
  const float logits[5] = {0.f, 3.f, 3.f, -2.f, 1.f};
  uint64_t rng = 99;
  pk::SamplerConfig greedy;
  CHECK(pk::sample_token(logits, 5, greedy, rng) == 1);
  pk::SamplerConfig hot;
  hot.temperature = 1.f;
  hot.top_p = 0.5f;
  int seen[5] = {0};
  for (int i = 0; i < 2000; ++i) seen[pk::sample_token(logits, 5, hot, rng)]++;
  CHECK(seen[0] == 0 && seen[3] == 0 && seen[4] == 0 && seen[1] > 0);
  // min-p: only candidates within a factor of the best survive (e^-2 = 0.135 of the best for token 4, e^-3 for token 0)
  pk::SamplerConfig mp;
  mp.temperature = 1.f;
  mp.min_p = 0.1f;
  int seen2[5] = {0};
  for (int i = 0; i < 4000; ++i) seen2[pk::sample_token(logits, 5, mp, rng)]++;
  CHECK(seen2[0] == 0 && seen2[3] == 0 && seen2[4] > 0 && seen2[1] > 0 && seen2[2] > 0);
  // penalties: token 1 was generated twice and token 2 once; the greedy pick moves to the untouched runner-up
  pk::SamplerConfig pen;
  pen.frequency_penalty = 0.5f;
  pen.presence_penalty = 0.25f;
  pen.repetition_penalty = 2.f;
  CHECK(pen.has_penalties() && !greedy.has_penalties());
  float l2[5] = {0.f, 3.f, 3.f, -2.f, 1.f};
  pk::apply_penalties(l2, 5, {1, 2, 1, 77, -3}, pen);
  CHECK(std::fabs(l2[1] - (1.5f - 1.0f - 0.25f)) < 1e-6f && std::fabs(l2[2] - (1.5f - 0.5f - 0.25f)) < 1e-6f && l2[0] == 0.f && l2[4] == 1.f);
  CHECK(pk::sample_token(l2, 5, pen, rng) == 4);
  // log-probabilities: log-softmax entry of the chosen token and the k largest, ties to the lower id
  pk::TokenLogprobs lp;
  pk::token_logprobs(logits, 5, 4, 3, &lp);
  const double lse = std::log(std::exp(0.0) + 2 * std::exp(3.0) + std::exp(-2.0) + std::exp(1.0));
  CHECK(std::fabs(lp.chosen - (float)(1.0 - lse)) < 1e-5f && lp.top.size() == 3);
  CHECK(lp.top[0].first == 1 && lp.top[1].first == 2 && lp.top[2].first == 4 && std::fabs(lp.top[0].second - (float)(3.0 - lse)) < 1e-5f);
  pk::token_logprobs(logits, 5, 9, 3, &lp);
  CHECK(lp.top.empty() && lp.chosen == 0.f);          // a token outside the vocabulary reports nothing
  float l3[2] = {-1.f, -4.f};
  pk::apply_penalties(l3, 2, {0}, pen);
  CHECK(std::fabs(l3[0] - (-2.f - 0.5f - 0.25f)) < 1e-6f && l3[1] == -4.f);    // a negative logit is multiplied
  return 0;
}

static int test_control_plane(const std::string& scratch) {
  const int world = 3;
  std::vector<std::vector<std::vector<uint8_t>>> got(world);
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r)
    th.emplace_back([&, r] { got[r] = pk::file_rendezvous(scratch + "/rdv", r, world, std::vector<uint8_t>(64, (uint8_t)(r + 1)), 20000, 5); });
  for (auto& t : th) t.join();
  for (int r = 0; r < world; ++r)
    for (int q = 0; q < world; ++q) CHECK(got[r][q].size() == 64 && got[r][q][0] == q + 1);
  for (int r = 0; r < world; ++r) pk::file_rendezvous_cleanup(scratch + "/rdv", r);
  // a rank that never arrives: the others give up with an error instead of waiting for ever
  bool threw = false;
  try {
    pk::file_rendezvous(scratch + "/rdv_missing", 0, 2, std::vector<uint8_t>(64, 1), 300, 5);
  } catch (const std::exception& e) {
    threw = std::string(e.what()).find("never published") != std::string::npos;
  }
  CHECK(threw);
  pk::file_rendezvous_cleanup(scratch + "/rdv_missing", 0);
  // command channel: rank 0 drives two workers; when rank 0 goes away the workers' receive() ends
  std::atomic<int> received{0}, eof{0};
  std::vector<std::thread> workers;
  for (int r = 1; r < world; ++r)
    workers.emplace_back([&, r] {
      pk::CmdChannel ch(scratch + "/cmd.sock", r, world, 400, 10);
      pk::CmdChannel::Message m;
      while (ch.receive(m)) {
        if (m.op == 7 && m.payload.size() == 3 && m.payload[2] == 30) received++;
      }
      eof++;
    });
  {
    pk::CmdChannel ch0(scratch + "/cmd.sock", 0, world, 400, 10);
    pk::CmdChannel::Message m;
    m.op = 7;
    m.payload = {10, 20, 30};
    for (int i = 0; i < 5; ++i) ch0.broadcast(m);
  }   // rank 0 closes its sockets here
  for (auto& t : workers) t.join();
  CHECK(received == 10 && eof == 2);
  // a worker that hangs up makes the next broadcast fail loudly
  threw = false;
  {
    std::thread w([&] { pk::CmdChannel ch(scratch + "/cmd2.sock", 1, 2, 400, 10); });
    pk::CmdChannel ch0(scratch + "/cmd2.sock", 0, 2, 400, 10);
    w.join();
    pk::CmdChannel::Message m;
    m.op = 1;
    m.payload.assign(1 << 16, 5);
    try {
      for (int i = 0; i < 50; ++i) ch0.broadcast(m);
    } catch (const std::exception&) {
      threw = true;
    }
  }
  CHECK(threw);
  return 0;
}

static int test_protocol() {
  const int world = 4, iters = 300;
  const size_t n = 257;
  std::vector<std::unique_ptr<pk::HostArena>> own;
  std::vector<pk::HostArena*> arenas;
  for (int r = 0; r < world; ++r) {
    own.push_back(std::make_unique<pk::HostArena>(world, n));
    arenas.push_back(own.back().get());
  }
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r)
    th.emplace_back([&, r] {
      std::vector<float> in(n), out(n);
      for (int it = 0; it < iters; ++it) {
        for (size_t i = 0; i < n; ++i) in[i] = (float)(r + 1) * (float)(it % 7 + 1) + (float)(i % 3);
        if ((it + r) % 5 == 0) std::this_thread::sleep_for(std::chrono::microseconds(200));   // ranks drift apart
        if (!pk::host_allreduce(arenas, r, in.data(), out.data(), n, 20000)) bad++;
        for (size_t i = 0; i < n; ++i) {
          const float want = 10.f * (float)(it % 7 + 1) + 4.f * (float)(i % 3);
          if (std::fabs(out[i] - want) > 1e-3f) bad++;
        }
      }
    });
  for (auto& t : th) t.join();
  CHECK(bad == 0);
  // rank 3 stays away: the others notice within their budget and say so through the status word
  std::vector<std::unique_ptr<pk::HostArena>> own2;
  std::vector<pk::HostArena*> arenas2;
  for (int r = 0; r < world; ++r) {
    own2.push_back(std::make_unique<pk::HostArena>(world, n));
    arenas2.push_back(own2.back().get());
  }
  std::atomic<int> timed_out{0};
  th.clear();
  for (int r = 0; r < world - 1; ++r)
    th.emplace_back([&, r] {
      std::vector<float> in(n, 1.f), out(n);
      if (!pk::host_allreduce(arenas2, r, in.data(), out.data(), n, 100)) timed_out++;
    });
  for (auto& t : th) t.join();
  CHECK(timed_out == world - 1 && arenas2[0]->status.load() == 1);
  return 0;
}

// In-switch all-reduce: one-shot and two-shot calls mixed, ranks drifting apart; then a rank that never joins.
static int test_multimem_protocol() {
  const int world = 4, iters = 300;
  const size_t n = 203;
  std::vector<std::unique_ptr<pk::HostMmBuffer>> own;
  std::vector<pk::HostMmBuffer*> bufs;
  for (int r = 0; r < world; ++r) {
    own.push_back(std::make_unique<pk::HostMmBuffer>(world, n));
    bufs.push_back(own.back().get());
  }
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r)
    th.emplace_back([&, r] {
      std::vector<float> in(n), out(n);
      for (int it = 0; it < iters; ++it) {
        for (size_t i = 0; i < n; ++i) in[i] = (float)(r + 1) * (float)(it % 7 + 1) + (float)(i % 3);
        if ((it + r) % 5 == 0) std::this_thread::sleep_for(std::chrono::microseconds(200));
        const bool two_shot = (it % 3) != 0;            // the same schedule on every rank, both kinds on both data sets
        if (!pk::host_mm_allreduce(bufs, r, in.data(), out.data(), n, two_shot, 20000)) bad++;
        for (size_t i = 0; i < n; ++i) {
          const float want = 10.f * (float)(it % 7 + 1) + 4.f * (float)(i % 3);
          if (std::fabs(out[i] - want) > 1e-3f) bad++;
        }
      }
    });
  for (auto& t : th) t.join();
  CHECK(bad == 0);
  std::vector<std::unique_ptr<pk::HostMmBuffer>> own2;
  std::vector<pk::HostMmBuffer*> bufs2;
  for (int r = 0; r < world; ++r) {
    own2.push_back(std::make_unique<pk::HostMmBuffer>(world, n));
    bufs2.push_back(own2.back().get());
  }
  std::atomic<int> timed_out{0};
  th.clear();
  for (int r = 0; r < world - 1; ++r)
    th.emplace_back([&, r] {
      std::vector<float> in(n, 1.f), out(n);
      if (!pk::host_mm_allreduce(bufs2, r, in.data(), out.data(), n, true, 100)) timed_out++;
    });
  for (auto& t : th) t.join();
  CHECK(timed_out == world - 1 && bufs2[0]->status.load() == 1);
  return 0;
}

// Block counters of the peer all-reduce kernel when blocks skip their wait (status word already set): with one shared
// counter the publish fires before every block has stored, or never; with one counter per pass it fires exactly when
// the last block has stored.
static int test_block_counters() {
  using pk::BlockEvent;
  // grid 3: b0 stores, b0 leaves (no wait: failed state), b1 stores -> a shared counter says "3 of 3" with b2 missing
  const std::vector<BlockEvent> a = {{0, 1}, {0, 2}, {1, 1}, {1, 2}, {2, 1}, {2, 2}};
  CHECK(pk::stored_at_publish(3, a, false) == 2);
  CHECK(pk::stored_at_publish(3, a, true) == 3);
  // grid 2: b0 stores, b0 leaves, b1 stores -> the shared counter jumps from 2 (a second-pass increment) to 3: never published
  const std::vector<BlockEvent> b = {{0, 1}, {0, 2}, {1, 1}, {1, 2}};
  CHECK(pk::stored_at_publish(2, b, false) == -1);
  CHECK(pk::stored_at_publish(2, b, true) == 2);
  // the healthy order is fine either way
  const std::vector<BlockEvent> c = {{0, 1}, {1, 1}, {2, 1}, {0, 2}, {1, 2}, {2, 2}};
  CHECK(pk::stored_at_publish(3, c, false) == 3 && pk::stored_at_publish(3, c, true) == 3);
  return 0;
}

// Prefix reuse decisions: live continuation, roll back to a stored state, start from zero; snapshot placement and eviction.
static int test_prefix_plan() {
  using pk::PrefixDecision;
  const std::vector<int> hist = {1, 2, 3, 4, 5, 6, 7, 8};   // the engine has consumed 8 tokens and stands at position 8
  const std::vector<int> snaps = {4, 6, 8};
  {  // the new prompt extends the whole consumed sequence: continue live, nothing restored
    const int p[] = {1, 2, 3, 4, 5, 6, 7, 8, 9, 10};
    const PrefixDecision d = pk::plan_prefix(hist, 8, snaps, p, 10);
    CHECK(d.source == PrefixDecision::kLive && d.resume_pos == 8 && d.matched == 8);
  }
  {  // the same prompt again: one token must still run, so the state at 8 is too far; the one at 6 serves
    const int p[] = {1, 2, 3, 4, 5, 6, 7, 8};
    const PrefixDecision d = pk::plan_prefix(hist, 8, snaps, p, 8);
    CHECK(d.source == PrefixDecision::kSnapshot && d.resume_pos == 6 && d.snapshot_index == 1 && d.matched == 8);
  }
  {  // divergence at position 5: roll back to the state stored at 4
    const int p[] = {1, 2, 3, 4, 5, 99, 98, 97};
    const PrefixDecision d = pk::plan_prefix(hist, 8, snaps, p, 8);
    CHECK(d.source == PrefixDecision::kSnapshot && d.resume_pos == 4 && d.matched == 5);
  }
  {  // divergence before the first stored state, or no state at all: from zero
    const int p[] = {1, 2, 3, 77};
    CHECK(pk::plan_prefix(hist, 8, snaps, p, 4).source == PrefixDecision::kEmpty);
    const int q[] = {1, 2, 3, 4, 5, 6};
    CHECK(pk::plan_prefix(hist, 8, {}, q, 6).source == PrefixDecision::kEmpty);
    CHECK(pk::plan_prefix({}, 0, {}, q, 6).resume_pos == 0);
  }
  {  // a shorter history than the live position (state restored by other means) can only match what it records
    const int p[] = {1, 2, 3, 4, 5};
    const PrefixDecision d = pk::plan_prefix({1, 2}, 8, {2}, p, 5);
    CHECK(d.matched == 2 && d.source == PrefixDecision::kSnapshot && d.resume_pos == 2);
  }
  CHECK((pk::snapshot_points(0, 10, 4) == std::vector<int>{4, 8, 10}));
  CHECK((pk::snapshot_points(4, 8, 4) == std::vector<int>{8}));
  CHECK((pk::snapshot_points(3, 9, 0) == std::vector<int>{9}));
  CHECK(pk::snapshot_points(5, 5, 4).empty());
  // eviction: request boundaries (not multiples of the interval) go first, oldest first; else the oldest of all
  CHECK(pk::snapshot_to_evict({4, 8, 10, 13}, {1, 2, 4, 3}, 4) == 3);
  CHECK(pk::snapshot_to_evict({4, 8, 12}, {5, 2, 9}, 4) == 1);
  return 0;
}

// Draft-length policy of speculative decode: a whole request simulated on the host.
static int test_spec_policy() {
  using pk::drafts_this_round;
  using pk::next_draft_len;
  CHECK(next_draft_len(1, 1, 1, 4) == 2 && next_draft_len(2, 2, 2, 4) == 4 && next_draft_len(4, 4, 4, 4) == 4);   // doubles up to the limit
  CHECK(next_draft_len(4, 4, 0, 4) == 1 && next_draft_len(4, 4, 1, 4) == 2 && next_draft_len(4, 4, 3, 4) == 2);   // max(1, min(K/2, ok+1))
  CHECK(next_draft_len(1, 1, 0, 4) == 1 && next_draft_len(7, 7, 6, 7) == 3);
  CHECK(next_draft_len(4, 2, 2, 4) == 4);   // a round cut short by the end of the request still counts as accepted
  CHECK(drafts_this_round(4, 10, 4) == 4 && drafts_this_round(4, 3, 4) == 2 && drafts_this_round(4, 1, 4) == 0 && drafts_this_round(2, 9, 1) == 1);
  // every request length ends exactly, whatever the drafts are worth: perfect drafts, useless drafts, alternating
  for (int pattern = 0; pattern < 3; ++pattern)
    for (int steps = 1; steps <= 40; ++steps) {
      int produced = 0, K = 1, rounds = 0;
      while (produced < steps) {
        const int k = drafts_this_round(K, steps - produced, 7);
        if (k == 0) {
          produced += 1;   // plain step
          continue;
        }
        const int accepted = pattern == 0 ? k : pattern == 1 ? 0 : (rounds & 1 ? k : k / 2);
        produced += accepted + 1;
        K = next_draft_len(K, k, accepted, 7);
        CHECK(K >= 1 && K <= 7);
        ++rounds;
      }
      CHECK(produced == steps);
    }
  return 0;
}

int main(int argc, char** argv) {
  if (argc < 4) {
    std::fprintf(stderr, "usage: host_selftest file.gguf safetensors_dir scratch_dir [tokenizer.gguf]\n");
    return 2;
  }
  try {
    if (test_json()) return 1;
    if (test_readers(argv[1], argv[2])) return 1;
    if (test_qwen_audit(argv[2])) return 1;
    if (test_safetensors_rejects_hostile_headers(argv[3])) return 1;
    if (test_weight_source_and_dsv4_config(argv[1], argv[2])) return 1;
    if (argc > 4 && test_tokenizer(argv[4])) return 1;
    if (test_sampler()) return 1;
    if (test_control_plane(argv[3])) return 1;
    if (test_protocol()) return 1;
    if (test_multimem_protocol()) return 1;
    if (test_block_counters()) return 1;
    if (test_prefix_plan()) return 1;
    if (test_spec_policy()) return 1;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "host_selftest: unexpected exception: %s\n", e.what());
    return 1;
  }
  std::printf("host_selftest=ok\n");
  return 0;
}
