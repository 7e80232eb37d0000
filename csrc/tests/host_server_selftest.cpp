// The OpenAI front end (HTTP, SSE, request loop, log-probability reports, worker engine) with its scripted engine or a
// Python model worker, as a small program of its own so that it can be built with AddressSanitizer + UBSan without the
// GPU engine. tests/test_host_sanitizers.py drives it over HTTP.
//   host_server_selftest PYTHON scripted SCRIPT | host_server_selftest PYTHON worker SCRIPT
#include <cstdio>
#include <string>
#include <vector>

#include "../engine/http_server.hpp"
#include "../engine/openai_server.hpp"

int main(int argc, char** argv) {
  if (argc < 4) {
    std::fprintf(stderr, "usage: host_server_selftest PYTHON scripted|worker SCRIPT\n");
    return 2;
  }
  try {
    const std::string python = argv[1], mode = argv[2], script = argv[3];
    std::unique_ptr<pk::TokenEngine> eng;
    if (mode == "worker")
      eng = pk::make_worker_engine({python, "-m", "pocketllm_b200.server.model_worker", "--model", "scripted", "--script", script, "--max-context", "512"});
    else
      eng = pk::make_scripted_engine(script, 512);
    pk::Sidecar sidecar({python, "-m", "pocketllm_b200.server.cpp_sidecar", "--tokenizer", "chars", "--chat-format", "dsv4"});
    pk::HttpServer http("127.0.0.1", 0);
    std::printf("openai_server_listening host=127.0.0.1 port=%d engine=%s\n", http.port(), mode.c_str());
    std::fflush(stdout);
    pk::OpenAIServerOptions so;
    so.model_name = "selftest";
    so.allow_shutdown = true;
    pk::run_openai_server(http, *eng, sidecar, so);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "host_server_selftest: %s\n", e.what());
    return 1;
  }
  std::printf("host_server_selftest=ok\n");
  return 0;
}
