// Single-threaded epoll HTTP/1.1 + WebSocket server for the control plane. Requests are small JSON bodies and uploads of
// a few MB; every handler runs to completion on the loop thread, so handlers must not block (the worker driver runs on
// its own thread and wakes the loop through an eventfd when there is something to push to WebSocket clients).
#pragma once
#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace mdb {
namespace http {

// ---- SHA-1 and base64 (only for the WebSocket accept key) -----------------------------------------------------------
inline std::string sha1(const std::string& in) {
  uint32_t h[5] = {0x67452301u, 0xEFCDAB89u, 0x98BADCFEu, 0x10325476u, 0xC3D2E1F0u};
  std::string m = in;
  uint64_t bits = static_cast<uint64_t>(in.size()) * 8;
  m += static_cast<char>(0x80);
  while (m.size() % 64 != 56) m += static_cast<char>(0);
  for (int i = 7; i >= 0; --i) m += static_cast<char>((bits >> (8 * i)) & 0xFF);
  auto rol = [](uint32_t v, int s) { return (v << s) | (v >> (32 - s)); };
  for (size_t off = 0; off < m.size(); off += 64) {
    uint32_t w[80];
    for (int i = 0; i < 16; ++i)
      w[i] = (static_cast<uint32_t>(static_cast<unsigned char>(m[off + 4 * i])) << 24) |
             (static_cast<uint32_t>(static_cast<unsigned char>(m[off + 4 * i + 1])) << 16) |
             (static_cast<uint32_t>(static_cast<unsigned char>(m[off + 4 * i + 2])) << 8) |
             static_cast<uint32_t>(static_cast<unsigned char>(m[off + 4 * i + 3]));
    for (int i = 16; i < 80; ++i) w[i] = rol(w[i - 3] ^ w[i - 8] ^ w[i - 14] ^ w[i - 16], 1);
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4];
    for (int i = 0; i < 80; ++i) {
      uint32_t f, k;
      if (i < 20) { f = (b & c) | (~b & d); k = 0x5A827999u; }
      else if (i < 40) { f = b ^ c ^ d; k = 0x6ED9EBA1u; }
      else if (i < 60) { f = (b & c) | (b & d) | (c & d); k = 0x8F1BBCDCu; }
      else { f = b ^ c ^ d; k = 0xCA62C1D6u; }
      uint32_t t = rol(a, 5) + f + e + k + w[i];
      e = d; d = c; c = rol(b, 30); b = a; a = t;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e;
  }
  std::string out(20, '\0');
  for (int i = 0; i < 5; ++i)
    for (int j = 0; j < 4; ++j) out[4 * i + j] = static_cast<char>((h[i] >> (24 - 8 * j)) & 0xFF);
  return out;
}
inline std::string base64(const std::string& in) {
  static const char* tbl = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
  std::string out;
  size_t i = 0;
  for (; i + 2 < in.size(); i += 3) {
    uint32_t v = (static_cast<unsigned char>(in[i]) << 16) | (static_cast<unsigned char>(in[i + 1]) << 8) | static_cast<unsigned char>(in[i + 2]);
    out += tbl[(v >> 18) & 63]; out += tbl[(v >> 12) & 63]; out += tbl[(v >> 6) & 63]; out += tbl[v & 63];
  }
  if (i + 1 == in.size()) {
    uint32_t v = static_cast<unsigned char>(in[i]) << 16;
    out += tbl[(v >> 18) & 63]; out += tbl[(v >> 12) & 63]; out += "==";
  } else if (i + 2 == in.size()) {
    uint32_t v = (static_cast<unsigned char>(in[i]) << 16) | (static_cast<unsigned char>(in[i + 1]) << 8);
    out += tbl[(v >> 18) & 63]; out += tbl[(v >> 12) & 63]; out += tbl[(v >> 6) & 63]; out += '=';
  }
  return out;
}
inline std::string base64_decode(const std::string& in) {
  std::string out;
  uint32_t acc = 0;
  int bits = 0;
  for (unsigned char c : in) {
    int v;
    if (c >= 'A' && c <= 'Z') v = c - 'A';
    else if (c >= 'a' && c <= 'z') v = c - 'a' + 26;
    else if (c >= '0' && c <= '9') v = c - '0' + 52;
    else if (c == '+' || c == '-') v = 62;
    else if (c == '/' || c == '_') v = 63;
    else continue;
    acc = (acc << 6) | static_cast<uint32_t>(v);
    bits += 6;
    if (bits >= 8) { bits -= 8; out += static_cast<char>((acc >> bits) & 0xFF); }
  }
  return out;
}
inline std::string url_decode(const std::string& s) {
  std::string o;
  for (size_t i = 0; i < s.size(); ++i) {
    if (s[i] == '%' && i + 2 < s.size() + 0 && isxdigit(static_cast<unsigned char>(s[i + 1])) && isxdigit(static_cast<unsigned char>(s[i + 2]))) {
      o += static_cast<char>(strtol(s.substr(i + 1, 2).c_str(), nullptr, 16));
      i += 2;
    } else if (s[i] == '+') o += ' ';
    else o += s[i];
  }
  return o;
}

struct Request {
  std::string method, path, query_string, body;
  std::map<std::string, std::string> headers;   // lower-cased names
  std::map<std::string, std::string> query;
  std::string header(const std::string& k) const { auto it = headers.find(k); return it == headers.end() ? "" : it->second; }
  std::string param(const std::string& k) const { auto it = query.find(k); return it == query.end() ? "" : it->second; }
};
struct Response {
  int status = 200;
  std::string content_type = "application/json";
  std::string body;
  bool upgrade_ws = false;            // handler accepted a WebSocket: the loop completes the handshake
  std::string ws_topic;               // what the socket subscribes to (a job id)
};

inline const char* reason(int s) {
  switch (s) {
    case 200: return "OK"; case 201: return "Created"; case 204: return "No Content"; case 400: return "Bad Request";
    case 404: return "Not Found"; case 405: return "Method Not Allowed"; case 409: return "Conflict";
    case 413: return "Payload Too Large"; case 422: return "Unprocessable Entity"; case 500: return "Internal Server Error";
    case 501: return "Not Implemented"; case 503: return "Service Unavailable"; default: return "Status";
  }
}

inline std::string ws_frame(const std::string& payload, int opcode = 1) {
  std::string f;
  f += static_cast<char>(0x80 | opcode);
  if (payload.size() < 126) f += static_cast<char>(payload.size());
  else if (payload.size() < 65536) { f += static_cast<char>(126); f += static_cast<char>(payload.size() >> 8); f += static_cast<char>(payload.size() & 0xFF); }
  else { f += static_cast<char>(127); for (int i = 7; i >= 0; --i) f += static_cast<char>((static_cast<uint64_t>(payload.size()) >> (8 * i)) & 0xFF); }
  return f + payload;
}

class Server {
 public:
  using Handler = std::function<void(const Request&, Response&)>;
  // called on the loop thread after the handshake and whenever wake() was signalled; returns frames to send, sets done
  using WsPump = std::function<std::vector<std::string>(const std::string& topic, size_t* cursor, bool* done)>;

  size_t max_body = 64u << 20;

  bool listen_on(int port, std::string* err) {
    lfd_ = socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
    if (lfd_ < 0) { *err = strerror(errno); return false; }
    int one = 1;
    setsockopt(lfd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    a.sin_port = htons(static_cast<uint16_t>(port));
    if (bind(lfd_, reinterpret_cast<sockaddr*>(&a), sizeof a) != 0 || listen(lfd_, 128) != 0) { *err = strerror(errno); return false; }
    socklen_t len = sizeof a;
    getsockname(lfd_, reinterpret_cast<sockaddr*>(&a), &len);
    port_ = ntohs(a.sin_port);
    ep_ = epoll_create1(EPOLL_CLOEXEC);
    wake_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    add(lfd_, EPOLLIN);
    add(wake_, EPOLLIN);
    return true;
  }
  int port() const { return port_; }
  void wake() { uint64_t v = 1; ssize_t r = write(wake_, &v, sizeof v); (void)r; }   // any thread
  void stop() { stop_ = true; wake(); }

  void run(const Handler& handler, const WsPump& pump) {
    epoll_event evs[64];
    while (!stop_) {
      int n = epoll_wait(ep_, evs, 64, 1000);
      for (int i = 0; i < n; ++i) {
        int fd = evs[i].data.fd;
        if (fd == lfd_) { accept_all(); continue; }
        if (fd == wake_) { uint64_t v; while (read(wake_, &v, sizeof v) > 0) {} continue; }
        auto it = conns_.find(fd);
        if (it == conns_.end()) continue;
        Conn& c = *it->second;
        if (evs[i].events & (EPOLLHUP | EPOLLERR)) { drop(fd); continue; }
        if (evs[i].events & EPOLLIN) { if (!on_read(c, handler)) { drop(fd); continue; } }
        if (evs[i].events & EPOLLOUT) { if (!flush(c)) { drop(fd); continue; } }
      }
      // push pending events to every WebSocket client (cheap: a handful of sockets)
      std::vector<int> closing;
      for (auto& kv : conns_) {
        Conn& c = *kv.second;
        if (!c.ws) continue;
        bool done = false;
        for (auto& frame : pump(c.topic, &c.cursor, &done)) c.out += ws_frame(frame);
        if (done && !c.close_sent) { c.out += ws_frame(std::string("\x03\xe8", 2), 8); c.close_sent = true; c.close_after_flush = true; }
        if (!flush(c)) closing.push_back(kv.first);
      }
      for (int fd : closing) drop(fd);
    }
    for (auto& kv : conns_) close(kv.first);
    conns_.clear();
    close(lfd_); close(ep_); close(wake_);
  }

 private:
  struct Conn {
    int fd;
    std::string in, out;
    bool ws = false, close_after_flush = false, close_sent = false;
    std::string topic;
    size_t cursor = 0;
  };
  void add(int fd, uint32_t ev) { epoll_event e{}; e.events = ev; e.data.fd = fd; epoll_ctl(ep_, EPOLL_CTL_ADD, fd, &e); }
  void mod(int fd, uint32_t ev) { epoll_event e{}; e.events = ev; e.data.fd = fd; epoll_ctl(ep_, EPOLL_CTL_MOD, fd, &e); }
  void drop(int fd) { epoll_ctl(ep_, EPOLL_CTL_DEL, fd, nullptr); close(fd); conns_.erase(fd); }
  void accept_all() {
    while (true) {
      int fd = accept4(lfd_, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
      if (fd < 0) break;
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      auto c = std::make_unique<Conn>();
      c->fd = fd;
      conns_[fd] = std::move(c);
      add(fd, EPOLLIN);
    }
  }
  bool flush(Conn& c) {
    while (!c.out.empty()) {
      ssize_t w = send(c.fd, c.out.data(), c.out.size(), MSG_NOSIGNAL);
      if (w < 0) {
        if (errno == EAGAIN) { mod(c.fd, EPOLLIN | EPOLLOUT); return true; }
        if (errno == EINTR) continue;
        return false;
      }
      c.out.erase(0, static_cast<size_t>(w));
    }
    mod(c.fd, EPOLLIN);
    return !c.close_after_flush;
  }
  bool on_read(Conn& c, const Handler& handler) {
    char buf[16384];
    while (true) {
      ssize_t n = recv(c.fd, buf, sizeof buf, 0);
      if (n == 0) return false;
      if (n < 0) { if (errno == EAGAIN) break; if (errno == EINTR) continue; return false; }
      c.in.append(buf, static_cast<size_t>(n));
      if (c.in.size() > max_body + 65536) return false;
    }
    return c.ws ? on_ws_data(c) : on_http_data(c, handler);
  }
  bool on_ws_data(Conn& c) {
    while (c.in.size() >= 2) {
      unsigned char b0 = c.in[0], b1 = c.in[1];
      uint64_t len = b1 & 0x7F;
      size_t off = 2;
      if (len == 126) { if (c.in.size() < 4) return true; len = (static_cast<unsigned char>(c.in[2]) << 8) | static_cast<unsigned char>(c.in[3]); off = 4; }
      else if (len == 127) { if (c.in.size() < 10) return true; len = 0; for (int i = 0; i < 8; ++i) len = (len << 8) | static_cast<unsigned char>(c.in[2 + i]); off = 10; }
      bool masked = b1 & 0x80;
      if (len > (1u << 20)) return false;
      if (c.in.size() < off + (masked ? 4 : 0) + len) return true;
      std::string payload = c.in.substr(off + (masked ? 4 : 0), len);
      if (masked) for (size_t i = 0; i < payload.size(); ++i) payload[i] ^= c.in[off + (i & 3)];
      c.in.erase(0, off + (masked ? 4 : 0) + len);
      int op = b0 & 0x0F;
      if (op == 8) { if (!c.close_sent) { c.out += ws_frame(payload.substr(0, 2), 8); c.close_sent = true; } c.close_after_flush = true; return flush(c); }
      if (op == 9) { c.out += ws_frame(payload, 10); if (!flush(c)) return false; }
    }
    return true;
  }
  bool on_http_data(Conn& c, const Handler& handler) {
    while (true) {
      size_t he = c.in.find("\r\n\r\n");
      if (he == std::string::npos) return c.in.size() < 65536;
      Request rq;
      size_t le = c.in.find("\r\n");
      std::string start = c.in.substr(0, le);
      size_t s1 = start.find(' '), s2 = start.rfind(' ');
      if (s1 == std::string::npos || s2 <= s1) return false;
      rq.method = start.substr(0, s1);
      std::string target = start.substr(s1 + 1, s2 - s1 - 1);
      size_t q = target.find('?');
      rq.path = url_decode(target.substr(0, q));
      if (q != std::string::npos) {
        rq.query_string = target.substr(q + 1);
        size_t p = 0;
        while (p <= rq.query_string.size()) {
          size_t amp = rq.query_string.find('&', p);
          std::string kv = rq.query_string.substr(p, amp == std::string::npos ? std::string::npos : amp - p);
          size_t eq = kv.find('=');
          if (!kv.empty()) rq.query[url_decode(kv.substr(0, eq))] = eq == std::string::npos ? "" : url_decode(kv.substr(eq + 1));
          if (amp == std::string::npos) break;
          p = amp + 1;
        }
      }
      size_t pos = le + 2;
      while (pos < he) {
        size_t e = c.in.find("\r\n", pos);
        std::string line = c.in.substr(pos, e - pos);
        size_t colon = line.find(':');
        if (colon != std::string::npos) {
          std::string k = line.substr(0, colon), v = line.substr(colon + 1);
          for (auto& ch : k) ch = static_cast<char>(tolower(static_cast<unsigned char>(ch)));
          while (!v.empty() && v.front() == ' ') v.erase(0, 1);
          rq.headers[k] = v;
        }
        pos = e + 2;
      }
      size_t clen = 0;
      if (!rq.header("content-length").empty()) clen = static_cast<size_t>(strtoull(rq.header("content-length").c_str(), nullptr, 10));
      if (clen > max_body) { respond(c, 413, "application/json", "{\"error\":\"body too large\"}", false); return flush(c); }
      if (c.in.size() < he + 4 + clen) return true;
      rq.body = c.in.substr(he + 4, clen);
      c.in.erase(0, he + 4 + clen);
      Response rs;
      handler(rq, rs);
      if (rs.upgrade_ws) {
        std::string key = rq.header("sec-websocket-key");
        if (key.empty()) { respond(c, 400, "application/json", "{\"error\":\"missing Sec-WebSocket-Key\"}", false); return flush(c); }
        c.out += "HTTP/1.1 101 Switching Protocols\r\nUpgrade: websocket\r\nConnection: Upgrade\r\nSec-WebSocket-Accept: " +
                 base64(sha1(key + "258EAFA5-E914-47DA-95CA-C5AB0DC85B11")) + "\r\n\r\n";
        c.ws = true;
        c.topic = rs.ws_topic;
        return flush(c);
      }
      bool keep = lower_eq(rq.header("connection"), "close") ? false : true;
      respond(c, rs.status, rs.content_type, rs.body, keep);
      if (!flush(c)) return false;
      if (!keep) return false;
    }
  }
  static bool lower_eq(std::string a, const char* b) { for (auto& ch : a) ch = static_cast<char>(tolower(static_cast<unsigned char>(ch))); return a == b; }
  void respond(Conn& c, int status, const std::string& ctype, const std::string& body, bool keep) {
    c.out += "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + ctype +
             "\r\nContent-Length: " + std::to_string(body.size()) + "\r\nAccess-Control-Allow-Origin: *\r\nConnection: " +
             (keep ? "keep-alive" : "close") + "\r\n\r\n" + body;
    if (!keep) c.close_after_flush = true;
  }

  int lfd_ = -1, ep_ = -1, wake_ = -1, port_ = 0;
  bool stop_ = false;
  std::map<int, std::unique_ptr<Conn>> conns_;
};

}  // namespace http
}  // namespace mdb
