// OpenAI-compatible endpoint of the native engine: /health, /v1/models, /v1/chat/completions
// (JSON or server-sent events). Chat templating, tokenisation, incremental detokenisation with
// stop strings and tool-call / reasoning parsing run in a Python sidecar process that speaks JSON
// lines over pipes; token generation stays in this process.
// Roles in the reference: cpp_engine/src/openai_server.cpp (routes 444-446, streaming 338,
// context check 265) and cpp_engine/src/python_sidecar.cpp + cpp_sidecar.py.
#pragma once

#include <atomic>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "http_server.hpp"
#include "json.hpp"
#include "sampler.hpp"

namespace pk {

// Thrown by a TokenEngine when the result of a step must be discarded (for example a peer-memory wait that ran out
// on some rank): the request ends with HTTP 500 (or an error event on a stream), no further token of it is sent and the
// next request starts from a fresh state.
struct EngineStepFailed : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// What the server needs from a model.
class TokenEngine {
 public:
  virtual ~TokenEngine() = default;
  virtual int max_context() const = 0;
  // Starts a new request; returns the first generated token.
  virtual int prefill(const std::vector<int>& prompt, const SamplerConfig& sampler, uint64_t seed) = 0;
  // The token after the last one returned.
  virtual int next() = 0;
  // The request that prefill() started is over (all of its tokens were taken, or it was cut short): engines that run
  // ahead or in other processes settle here. Called once per started request.
  virtual void finish() {}
  // Log-probabilities of the step that produced the token returned last, when the request's sampler asked for them
  // (`SamplerConfig::logprobs >= 0`); false when this engine cannot report them.
  virtual bool last_logprobs(TokenLogprobs* out) {
    (void)out;
    return false;
  }
};

// Child process speaking one JSON object per line on stdin/stdout.
class Sidecar {
 public:
  explicit Sidecar(const std::vector<std::string>& argv);
  ~Sidecar();
  Json call(const Json& request);

 private:
  int to_child_ = -1, from_child_ = -1;
  int pid_ = -1;
  std::string pending_;
};

struct OpenAIServerOptions {
  std::string model_name = "pocketllm-b200";
  bool allow_shutdown = false;   // POST /shutdown ends serve() (used by tests)
};

// Blocks until stopped.
void run_openai_server(HttpServer& http, TokenEngine& engine, Sidecar& sidecar, const OpenAIServerOptions& opt);

// A model that lives in a child process (`python -m pocketllm_b200.server.model_worker ...`) and speaks JSON lines:
// prefill / next / log-probabilities are forwarded, a reply marked "lost" becomes EngineStepFailed. This is how the
// native front end serves the model families whose runtime is the Python one (DeepSeek-V4, the GGUF runtimes).
std::unique_ptr<TokenEngine> make_worker_engine(const std::vector<std::string>& argv);

// Deterministic stand-in for a model: replays `script` code points, then token 0 (EOS), for every request.
// The code point U+2620 in the script makes that step throw EngineStepFailed (to test the error path).
std::unique_ptr<TokenEngine> make_scripted_engine(const std::string& script, int max_context);

}  // namespace pk
