#include "openai_server.hpp"

#include <signal.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace pk {

// ---------------------------------------------------------------------------------------
// sidecar

Sidecar::Sidecar(const std::vector<std::string>& argv) {
  if (argv.empty()) throw std::runtime_error("sidecar: empty command");
  int in_pipe[2], out_pipe[2];
  if (pipe(in_pipe) != 0 || pipe(out_pipe) != 0) throw std::runtime_error("sidecar: pipe() failed");
  const pid_t pid = fork();
  if (pid < 0) throw std::runtime_error("sidecar: fork() failed");
  if (pid == 0) {
    dup2(in_pipe[0], 0);
    dup2(out_pipe[1], 1);
    close(in_pipe[0]);
    close(in_pipe[1]);
    close(out_pipe[0]);
    close(out_pipe[1]);
    std::vector<char*> args;
    for (const auto& a : argv) args.push_back(const_cast<char*>(a.c_str()));
    args.push_back(nullptr);
    execvp(args[0], args.data());
    std::perror("sidecar: exec");
    _exit(127);
  }
  close(in_pipe[0]);
  close(out_pipe[1]);
  to_child_ = in_pipe[1];
  from_child_ = out_pipe[0];
  pid_ = (int)pid;
  signal(SIGPIPE, SIG_IGN);
  const Json hello = call(Json::parse("{\"op\":\"hello\"}"));
  if (!hello.get_bool("ok", false)) throw std::runtime_error("sidecar: handshake failed");
}

Sidecar::~Sidecar() {
  if (to_child_ >= 0) {
    const char bye[] = "{\"op\":\"quit\"}\n";
    (void)!write(to_child_, bye, sizeof bye - 1);
    close(to_child_);
  }
  if (from_child_ >= 0) close(from_child_);
  if (pid_ > 0) {
    int st = 0;
    for (int i = 0; i < 50; ++i) {          // up to ~5 s for a clean exit, then end exactly this child
      if (waitpid(pid_, &st, WNOHANG) == pid_) return;
      usleep(100 * 1000);
    }
    kill(pid_, SIGKILL);
    waitpid(pid_, &st, 0);
  }
}

Json Sidecar::call(const Json& request) {
  std::string line = request.dump();
  line.push_back('\n');
  size_t off = 0;
  while (off < line.size()) {
    const ssize_t w = write(to_child_, line.data() + off, line.size() - off);
    if (w <= 0) throw std::runtime_error("sidecar: write failed (process gone?)");
    off += (size_t)w;
  }
  for (;;) {
    const size_t nl = pending_.find('\n');
    if (nl != std::string::npos) {
      const std::string reply = pending_.substr(0, nl);
      pending_.erase(0, nl + 1);
      return Json::parse(reply);
    }
    char buf[65536];
    const ssize_t n = read(from_child_, buf, sizeof buf);
    if (n <= 0) throw std::runtime_error("sidecar: closed its output");
    pending_.append(buf, (size_t)n);
  }
}

// ---------------------------------------------------------------------------------------
// scripted engine

namespace {
class ScriptedEngine : public TokenEngine {
 public:
  ScriptedEngine(const std::string& script, int max_context) : max_context_(max_context) {
    // UTF-8 -> code points
    for (size_t i = 0; i < script.size();) {
      const unsigned char c = (unsigned char)script[i];
      int len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
      int cp = len == 1 ? c : c & (0xff >> (len + 1));
      for (int k = 1; k < len && i + k < script.size(); ++k) cp = (cp << 6) | ((unsigned char)script[i + k] & 0x3f);
      cps_.push_back(cp);
      i += (size_t)len;
    }
  }
  int max_context() const override { return max_context_; }
  int prefill(const std::vector<int>&, const SamplerConfig& sc, uint64_t) override {
    pos_ = 0;
    top_k_ = sc.logprobs;
    return next();
  }
  int next() override {
    if (pos_ < cps_.size() && cps_[pos_] == 0x2620) {
      ++pos_;
      throw EngineStepFailed("scripted step failure");
    }
    last_ = pos_ < cps_.size() ? cps_[pos_++] : 0;
    return last_;
  }
  // a made-up distribution: the scripted token at ln(0.5), then its successors in code-point order at half of that each
  bool last_logprobs(TokenLogprobs* out) override {
    if (top_k_ < 0) return false;
    out->chosen = -0.6931472f;
    out->top.clear();
    for (int i = 0; i < top_k_; ++i) out->top.emplace_back(last_ + i, -0.6931472f * (float)(i + 1));
    return true;
  }

 private:
  std::vector<int> cps_;
  size_t pos_ = 0;
  int max_context_;
  int top_k_ = -1, last_ = 0;
};

std::string error_json(const std::string& msg, const std::string& type) {
  Json e = Json::object();
  e["message"] = Json(msg);
  e["type"] = Json(type);
  Json o = Json::object();
  o["error"] = e;
  return o.dump();
}

int64_t now_s() { return (int64_t)std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count(); }

}  // namespace

namespace {
class WorkerEngine : public TokenEngine {
 public:
  explicit WorkerEngine(const std::vector<std::string>& argv) : worker_(argv) {
    const Json hello = worker_.call(Json::parse("{\"op\":\"hello\"}"));
    max_context_ = (int)hello.get_int("max_context", 4096);
  }
  int max_context() const override { return max_context_; }
  int prefill(const std::vector<int>& prompt, const SamplerConfig& sc, uint64_t seed) override {
    Json req = Json::object();
    req["op"] = Json("prefill");
    req["tokens"] = Json::array();
    for (int t : prompt) req["tokens"].push_back(Json(t));
    Json s = Json::object();
    s["temperature"] = Json((double)sc.temperature);
    s["top_p"] = Json((double)sc.top_p);
    s["top_k"] = Json(sc.top_k);
    s["min_p"] = Json((double)sc.min_p);
    s["frequency_penalty"] = Json((double)sc.frequency_penalty);
    s["presence_penalty"] = Json((double)sc.presence_penalty);
    s["repetition_penalty"] = Json((double)sc.repetition_penalty);
    s["logprobs"] = Json(sc.logprobs);
    req["sampler"] = s;
    req["max_tokens"] = Json(sc.max_tokens);
    req["stop_token_ids"] = Json::array();
    for (int t : sc.stop_token_ids) req["stop_token_ids"].push_back(Json(t));
    req["seed"] = Json((int64_t)(seed & 0x7fffffffULL));
    return take(worker_.call(req));
  }
  int next() override { return take(worker_.call(Json::parse("{\"op\":\"next\"}"))); }
  void finish() override { worker_.call(Json::parse("{\"op\":\"end\"}")); }
  bool last_logprobs(TokenLogprobs* out) override {
    if (!have_lp_) return false;
    *out = lp_;
    return true;
  }

 private:
  int take(const Json& reply) {
    if (const Json* err = reply.find("error")) {
      if (reply.get_bool("lost", false)) throw EngineStepFailed(err->as_string());
      throw std::runtime_error(err->as_string());
    }
    have_lp_ = false;
    if (const Json* lp = reply.find("logprob")) {
      lp_.chosen = (float)lp->as_double();
      lp_.top.clear();
      if (const Json* top = reply.find("top"))
        for (const Json& e : top->items())
          if (e.items().size() == 2) lp_.top.emplace_back((int)e.items()[0].as_int(), (float)e.items()[1].as_double());
      have_lp_ = true;
    }
    return (int)reply.get_int("token", 0);
  }
  Sidecar worker_;
  int max_context_ = 4096;
  TokenLogprobs lp_;
  bool have_lp_ = false;
};
}  // namespace

std::unique_ptr<TokenEngine> make_worker_engine(const std::vector<std::string>& argv) { return std::make_unique<WorkerEngine>(argv); }

std::unique_ptr<TokenEngine> make_scripted_engine(const std::string& script, int max_context) {
  return std::make_unique<ScriptedEngine>(script, max_context);
}

// ---------------------------------------------------------------------------------------
// routes

void run_openai_server(HttpServer& http, TokenEngine& engine, Sidecar& sidecar, const OpenAIServerOptions& opt) {
  std::atomic<bool> stop{false};
  uint64_t counter = 0;
  auto handler = [&](const HttpRequest& req, HttpResponse& res) {
    if (req.method == "GET" && (req.path == "/health" || req.path == "/healthz")) {
      res.send(200, "application/json", "{\"status\":\"ok\"}");
      return;
    }
    if (req.method == "GET" && req.path == "/v1/models") {
      Json m = Json::object();
      m["id"] = Json(opt.model_name);
      m["object"] = Json("model");
      m["created"] = Json(now_s());
      m["owned_by"] = Json("pocketllm-b200");
      Json list = Json::object();
      list["object"] = Json("list");
      list["data"] = Json::array();
      list["data"].push_back(m);
      res.send(200, "application/json", list.dump());
      return;
    }
    if (req.method == "POST" && req.path == "/shutdown" && opt.allow_shutdown) {
      stop.store(true);
      res.send(200, "application/json", "{\"status\":\"stopping\"}");
      return;
    }
    if (req.path != "/v1/chat/completions") {
      res.send(404, "application/json", error_json("unknown route " + req.path, "invalid_request_error"));
      return;
    }
    if (req.method != "POST") {
      res.send(405, "application/json", error_json("use POST", "invalid_request_error"));
      return;
    }
    Json body;
    try {
      body = Json::parse(req.body);
      if (!body.is_object()) throw std::runtime_error("body must be a JSON object");
    } catch (const std::exception& e) {
      res.send(400, "application/json", error_json(std::string("invalid JSON: ") + e.what(), "invalid_request_error"));
      return;
    }
    Json begin = Json::object();
    begin["op"] = Json("begin");
    begin["body"] = body;
    const Json plan = sidecar.call(begin);
    if (!plan.get_bool("ok", false)) {
      res.send((int)plan.get_int("status", 400), "application/json",
               error_json(plan.get_string("error", "bad request"), "invalid_request_error"));
      return;
    }
    std::vector<int> prompt;
    for (const Json& t : plan.at("tokens").items()) prompt.push_back((int)t.as_int());
    const int max_tokens = (int)plan.get_int("max_tokens", 512);
    if ((int)prompt.size() + max_tokens > engine.max_context()) {
      res.send(400, "application/json",
               error_json("prompt (" + std::to_string(prompt.size()) + " tokens) plus max_tokens (" + std::to_string(max_tokens) +
                              ") exceeds the context of " + std::to_string(engine.max_context()) + " tokens",
                          "context_length_exceeded"));
      return;
    }
    std::vector<int> eos;
    for (const Json& t : plan.at("stop_token_ids").items()) eos.push_back((int)t.as_int());
    const bool stream = plan.get_bool("stream", false), include_usage = plan.get_bool("include_usage", false);
    SamplerConfig sc;
    sc.temperature = (float)plan.get_double("temperature", 0.0);
    sc.top_p = (float)plan.get_double("top_p", 1.0);
    sc.top_k = (int)plan.get_int("top_k", 0);
    sc.min_p = (float)plan.get_double("min_p", 0.0);
    sc.frequency_penalty = (float)plan.get_double("frequency_penalty", 0.0);
    sc.presence_penalty = (float)plan.get_double("presence_penalty", 0.0);
    sc.repetition_penalty = (float)plan.get_double("repetition_penalty", 1.0);
    sc.logprobs = (int)plan.get_int("logprobs", -1);
    sc.max_tokens = max_tokens;
    sc.stop_token_ids = eos;
    std::vector<std::pair<int, TokenLogprobs>> lps;      // generated tokens (no end-of-sequence token) with their log-probabilities
    const uint64_t seed = (uint64_t)plan.get_int("seed", 0) * 0x9E3779B97F4A7C15ULL + 0x1234567ULL;
    const std::string id = "chatcmpl-" + std::to_string(now_s()) + "-" + std::to_string(++counter);
    const int64_t created = now_s();

    auto chunk = [&](const Json& delta, const Json& finish) {
      Json c = Json::object();
      c["id"] = Json(id);
      c["object"] = Json("chat.completion.chunk");
      c["created"] = Json(created);
      c["model"] = Json(opt.model_name);
      Json choice = Json::object();
      choice["index"] = Json(0);
      choice["delta"] = delta;
      choice["finish_reason"] = finish;
      c["choices"] = Json::array();
      c["choices"].push_back(choice);
      return c.dump();
    };
    if (stream) {
      res.begin_sse();
      Json role = Json::object();
      role["role"] = Json("assistant");
      res.event(chunk(role, Json()));
    }
    int generated = 0;
    std::string finish = "length";
    int tok = 0;
    struct RequestEnd {
      TokenEngine& e;
      ~RequestEnd() {
        try {
          e.finish();
        } catch (...) {
        }
      }
    } request_end{engine};
    try {
      tok = engine.prefill(prompt, sc, seed);
    } catch (const std::exception& e) {
      // nothing has been sent yet when the request is not streamed; a stream gets an error event
      Json endq = Json::object();
      endq["op"] = Json("end");
      endq["finish_reason"] = Json("stop");
      sidecar.call(endq);
      const bool lost = dynamic_cast<const EngineStepFailed*>(&e) != nullptr;
      if (!stream) {
        res.send(lost ? 500 : 400, "application/json", error_json(e.what(), lost ? "engine_error" : "invalid_request_error"));
      } else {
        res.event(error_json(e.what(), lost ? "engine_error" : "invalid_request_error"));
        res.event("[DONE]");
        res.end_sse();
      }
      return;
    }
    bool step_lost = false, logprobs_refused = false;
    std::string step_error;
    while (true) {
      ++generated;
      bool is_eos = false;
      for (int e : eos) is_eos |= tok == e;
      if (is_eos) {
        finish = "stop";
        break;
      }
      if (sc.logprobs >= 0) {
        TokenLogprobs lp;
        if (!engine.last_logprobs(&lp)) {
          step_lost = true;
          step_error = "this engine does not report log-probabilities";
          logprobs_refused = true;
          break;
        }
        lps.emplace_back(tok, std::move(lp));
      }
      Json feed = Json::object();
      feed["op"] = Json("token");
      feed["token"] = Json(tok);
      const Json out = sidecar.call(feed);
      const std::string text = out.get_string("delta", "");
      if (stream && !text.empty()) {
        Json d = Json::object();
        d[out.get_string("channel", "content")] = Json(text);
        if (!res.event(chunk(d, Json()))) break;          // client went away
      }
      if (out.get_bool("stop", false)) {
        finish = "stop";
        break;
      }
      if (generated >= max_tokens) break;
      try {
        tok = engine.next();
      } catch (const std::exception& e) {
        // the step's result is gone (a rank timed out, or the engine refused): nothing of it is sent
        step_lost = true;
        step_error = e.what();
        break;
      }
    }
    if (step_lost) {
      Json endq = Json::object();
      endq["op"] = Json("end");
      endq["finish_reason"] = Json("stop");
      sidecar.call(endq);
      if (!stream) {
        res.send(logprobs_refused ? 400 : 500, "application/json", error_json(step_error, logprobs_refused ? "invalid_request_error" : "engine_error"));
      } else {
        res.event(error_json(step_error, "engine_error"));
        res.event("[DONE]");
        res.end_sse();
      }
      return;
    }
    Json endq = Json::object();
    endq["op"] = Json("end");
    endq["finish_reason"] = Json(finish);
    const Json fin = sidecar.call(endq);
    finish = fin.get_string("finish_reason", finish);
    Json usage = Json::object();
    usage["prompt_tokens"] = Json((int64_t)prompt.size());
    usage["completion_tokens"] = Json(generated);
    usage["total_tokens"] = Json((int64_t)prompt.size() + generated);
    if (stream) {
      const std::string tail = fin.get_string("tail", "");
      if (!tail.empty()) {
        Json d = Json::object();
        d[fin.get_string("channel", "content")] = Json(tail);
        res.event(chunk(d, Json()));
      }
      if (const Json* tc = fin.at("message").find("tool_calls")) {
        Json d = Json::object();
        d["tool_calls"] = *tc;
        res.event(chunk(d, Json()));
      }
      res.event(chunk(Json::object(), Json(finish)));
      if (include_usage) {
        Json u = Json::object();
        u["id"] = Json(id);
        u["object"] = Json("chat.completion.chunk");
        u["created"] = Json(created);
        u["model"] = Json(opt.model_name);
        u["choices"] = Json::array();
        u["usage"] = usage;
        res.event(u.dump());
      }
      res.event("[DONE]");
      res.end_sse();
      return;
    }
    Json out = Json::object();
    out["id"] = Json(id);
    out["object"] = Json("chat.completion");
    out["created"] = Json(created);
    out["model"] = Json(opt.model_name);
    Json choice = Json::object();
    choice["index"] = Json(0);
    choice["message"] = fin.at("message");
    choice["finish_reason"] = Json(finish);
    if (sc.logprobs >= 0) {
      // token texts come from the sidecar (one call for every id that appears)
      Json ask = Json::object();
      ask["op"] = Json("token_texts");
      ask["ids"] = Json::array();
      for (const auto& e : lps) {
        ask["ids"].push_back(Json(e.first));
        for (const auto& t : e.second.top) ask["ids"].push_back(Json(t.first));
      }
      const Json texts = sidecar.call(ask);
      size_t at = 0;
      auto entry = [&](float lp) {
        const std::string text = at < texts.at("texts").items().size() ? texts.at("texts").items()[at].as_string() : std::string();
        ++at;
        Json e = Json::object();
        e["token"] = Json(text);
        e["logprob"] = Json((double)lp);
        e["bytes"] = Json::array();
        for (unsigned char ch : text) e["bytes"].push_back(Json((int)ch));
        return e;
      };
      Json content = Json::array();
      for (const auto& e : lps) {
        Json one = entry(e.second.chosen);
        one["top_logprobs"] = Json::array();
        for (const auto& t : e.second.top) one["top_logprobs"].push_back(entry(t.second));
        content.push_back(one);
      }
      Json lpj = Json::object();
      lpj["content"] = content;
      choice["logprobs"] = lpj;
    }
    out["choices"] = Json::array();
    out["choices"].push_back(choice);
    out["usage"] = usage;
    res.send(200, "application/json", out.dump());
  };
  http.serve(handler, stop);
}

}  // namespace pk
