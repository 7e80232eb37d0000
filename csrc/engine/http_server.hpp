// Minimal blocking HTTP/1.1 server for the engine's OpenAI endpoint: one request in flight at a
// time (like the reference's server, cpp_engine/src/openai_server.cpp:179,264), JSON responses
// and chunked server-sent events. POSIX sockets only; no third-party code.
#pragma once

#include <atomic>
#include <functional>
#include <map>
#include <string>

namespace pk {

struct HttpRequest {
  std::string method, path, body;
  std::map<std::string, std::string> headers;   // lower-case names
};

class HttpResponse {
 public:
  explicit HttpResponse(int fd) : fd_(fd) {}
  // Complete response with a body.
  bool send(int status, const std::string& content_type, const std::string& body);
  // Streaming: begin_sse() once, event() per message, end_sse() at the end.
  bool begin_sse();
  bool event(const std::string& data);
  bool end_sse();
  bool started() const { return started_; }

 private:
  bool write_all(const char* p, size_t n);
  int fd_;
  bool started_ = false;
};

class HttpServer {
 public:
  // port 0 picks a free port; see port().
  HttpServer(const std::string& host, int port);
  ~HttpServer();
  int port() const { return port_; }
  using Handler = std::function<void(const HttpRequest&, HttpResponse&)>;
  // Serves until `stop` becomes true (checked between connections, once per second when idle).
  void serve(const Handler& handler, const std::atomic<bool>& stop);

 private:
  int listen_fd_ = -1, port_ = 0;
};

}  // namespace pk
