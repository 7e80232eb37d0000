#include "http_server.hpp"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace pk {
namespace {

const char* reason(int status) {
  switch (status) {
    case 200: return "OK";
    case 400: return "Bad Request";
    case 404: return "Not Found";
    case 405: return "Method Not Allowed";
    case 413: return "Payload Too Large";
    case 500: return "Internal Server Error";
    case 503: return "Service Unavailable";
    default: return "Status";
  }
}

constexpr size_t kMaxHeader = 64 * 1024, kMaxBody = 64u << 20;

bool read_request(int fd, HttpRequest& req, int& status) {
  std::string buf;
  char tmp[8192];
  size_t header_end = std::string::npos;
  while (header_end == std::string::npos) {
    const ssize_t n = recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) return false;
    buf.append(tmp, (size_t)n);
    header_end = buf.find("\r\n\r\n");
    if (header_end == std::string::npos && buf.size() > kMaxHeader) {
      status = 413;
      return true;
    }
  }
  const std::string head = buf.substr(0, header_end);
  size_t line_end = head.find("\r\n");
  const std::string first = head.substr(0, line_end);
  const size_t s1 = first.find(' '), s2 = first.rfind(' ');
  if (s1 == std::string::npos || s2 == s1) {
    status = 400;
    return true;
  }
  req.method = first.substr(0, s1);
  req.path = first.substr(s1 + 1, s2 - s1 - 1);
  const size_t q = req.path.find('?');
  if (q != std::string::npos) req.path.resize(q);
  size_t pos = line_end == std::string::npos ? head.size() : line_end + 2;
  while (pos < head.size()) {
    size_t e = head.find("\r\n", pos);
    if (e == std::string::npos) e = head.size();
    const std::string line = head.substr(pos, e - pos);
    const size_t c = line.find(':');
    if (c != std::string::npos) {
      std::string k = line.substr(0, c), v = line.substr(c + 1);
      std::transform(k.begin(), k.end(), k.begin(), [](unsigned char ch) { return (char)std::tolower(ch); });
      v.erase(0, v.find_first_not_of(" \t"));
      req.headers[k] = v;
    }
    pos = e + 2;
  }
  size_t want = 0;
  auto it = req.headers.find("content-length");
  if (it != req.headers.end()) want = (size_t)std::strtoull(it->second.c_str(), nullptr, 10);
  if (want > kMaxBody) {
    status = 413;
    return true;
  }
  req.body = buf.substr(header_end + 4);
  while (req.body.size() < want) {
    const ssize_t n = recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) return false;
    req.body.append(tmp, (size_t)n);
  }
  req.body.resize(want);
  return true;
}

}  // namespace

bool HttpResponse::write_all(const char* p, size_t n) {
  while (n > 0) {
    const ssize_t w = ::send(fd_, p, n, MSG_NOSIGNAL);
    if (w <= 0) return false;
    p += w;
    n -= (size_t)w;
  }
  return true;
}

bool HttpResponse::send(int status, const std::string& content_type, const std::string& body) {
  started_ = true;
  char head[512];
  const int n = std::snprintf(head, sizeof head,
                              "HTTP/1.1 %d %s\r\nContent-Type: %s\r\nContent-Length: %zu\r\nConnection: close\r\n\r\n", status,
                              reason(status), content_type.c_str(), body.size());
  return write_all(head, (size_t)n) && write_all(body.data(), body.size());
}

bool HttpResponse::begin_sse() {
  started_ = true;
  static const char head[] =
      "HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\n"
      "Connection: close\r\n\r\n";
  return write_all(head, sizeof head - 1);
}

bool HttpResponse::event(const std::string& data) {
  const std::string payload = "data: " + data + "\n\n";
  char len[32];
  const int n = std::snprintf(len, sizeof len, "%zx\r\n", payload.size());
  return write_all(len, (size_t)n) && write_all(payload.data(), payload.size()) && write_all("\r\n", 2);
}

bool HttpResponse::end_sse() { return write_all("0\r\n\r\n", 5); }

HttpServer::HttpServer(const std::string& host, int port) {
  listen_fd_ = socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) throw std::runtime_error("http: socket() failed");
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons((uint16_t)port);
  if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) throw std::runtime_error("http: bad host " + host);
  if (bind(listen_fd_, (sockaddr*)&addr, sizeof addr) != 0) throw std::runtime_error("http: bind failed on " + host + ":" + std::to_string(port));
  if (listen(listen_fd_, 16) != 0) throw std::runtime_error("http: listen failed");
  socklen_t len = sizeof addr;
  getsockname(listen_fd_, (sockaddr*)&addr, &len);
  port_ = ntohs(addr.sin_port);
}

HttpServer::~HttpServer() {
  if (listen_fd_ >= 0) close(listen_fd_);
}

void HttpServer::serve(const Handler& handler, const std::atomic<bool>& stop) {
  while (!stop.load()) {
    pollfd pfd{listen_fd_, POLLIN, 0};
    if (poll(&pfd, 1, 1000) <= 0) continue;
    const int fd = accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    timeval tv{30, 0};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    HttpRequest req;
    HttpResponse res(fd);
    int status = 0;
    if (read_request(fd, req, status)) {
      if (status != 0) {
        res.send(status, "application/json", "{\"error\":{\"message\":\"malformed or oversized request\",\"type\":\"invalid_request_error\"}}");
      } else {
        try {
          handler(req, res);
        } catch (const std::exception& e) {
          if (!res.started()) res.send(500, "application/json", std::string("{\"error\":{\"message\":\"internal error\",\"type\":\"server_error\"}}"));
          std::fprintf(stderr, "http: handler failed: %s\n", e.what());
        }
      }
    }
    shutdown(fd, SHUT_RDWR);
    close(fd);
  }
}

}  // namespace pk
