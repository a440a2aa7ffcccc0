// One worker process on the other end of an AF_UNIX stream socket pair. The child inherits its end as an open file
// descriptor whose number is appended to its argv. Lines are '\n' framed. A closed peer (recv() == 0) is an ordinary,
// typed outcome: the job in flight fails, the next job respawns the worker, the control plane keeps running.
// Swapping models = SIGKILL the child (process exit is the only reliable way to hand device memory back), wait for it,
// settle, spawn the next one (serenity-server/crates/ipc/src/lib.rs:34-250; serve/process_isolated_backend.mojo:22-174).
#pragma once
#include <fcntl.h>
#include <poll.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/types.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <string>
#include <vector>

namespace mdb {

class WorkerProc {
 public:
  enum Poll { Line, Idle, PeerClosed, IoError };

  ~WorkerProc() { kill_and_reap(); }

  // argv[0] is looked up on PATH. Returns false (and sets ``err``) if the pair or the fork fails; an exec failure shows
  // up as an immediate peer close.
  bool spawn(const std::vector<std::string>& argv, std::string* err) {
    int sv[2];
    if (socketpair(AF_UNIX, SOCK_STREAM, 0, sv) != 0) { *err = std::string("socketpair: ") + strerror(errno); return false; }
    std::vector<std::string> args = argv;
    args.push_back(std::to_string(sv[1]));
    std::vector<char*> cargs;
    for (auto& a : args) cargs.push_back(const_cast<char*>(a.c_str()));
    cargs.push_back(nullptr);
    pid_t pid = fork();
    if (pid < 0) { *err = std::string("fork: ") + strerror(errno); close(sv[0]); close(sv[1]); return false; }
    if (pid == 0) {
      close(sv[0]);
      int fl = fcntl(sv[1], F_GETFD);
      if (fl >= 0) fcntl(sv[1], F_SETFD, fl & ~FD_CLOEXEC);
      setpgid(0, 0);                       // own process group: the whole worker tree can be signalled at once
      execvp(cargs[0], cargs.data());
      _exit(127);
    }
    close(sv[1]);
    fcntl(sv[0], F_SETFL, fcntl(sv[0], F_GETFL) | O_NONBLOCK);
    fcntl(sv[0], F_SETFD, FD_CLOEXEC);
    fd_ = sv[0];
    pid_ = pid;
    peer_open_ = true;
    buf_.clear();
    return true;
  }

  bool alive() const { return pid_ > 0; }
  pid_t pid() const { return pid_; }

  bool send_line(const std::string& line, std::string* err) {
    std::string framed = line + "\n";
    size_t sent = 0;
    while (sent < framed.size()) {
      ssize_t w = send(fd_, framed.data() + sent, framed.size() - sent, MSG_NOSIGNAL);
      if (w < 0) {
        if (errno == EINTR) continue;
        if (errno == EAGAIN) { struct pollfd p{fd_, POLLOUT, 0}; poll(&p, 1, 1000); continue; }
        *err = std::string("send to worker failed: ") + strerror(errno);
        return false;
      }
      if (w == 0) { *err = "send returned 0 (peer closed)"; return false; }
      sent += static_cast<size_t>(w);
    }
    return true;
  }

  // Waits up to ``timeout_ms`` for one complete line.
  Poll next_line(std::string* line, int timeout_ms) {
    if (take_line(line)) return Line;
    if (!peer_open_) return PeerClosed;
    struct pollfd p{fd_, POLLIN, 0};
    int r = poll(&p, 1, timeout_ms);
    if (r == 0 || (r < 0 && errno == EINTR)) return Idle;
    if (r < 0) return IoError;
    char chunk[4096];
    ssize_t n = recv(fd_, chunk, sizeof chunk, 0);
    if (n == 0) { peer_open_ = false; return PeerClosed; }
    if (n < 0) return (errno == EAGAIN || errno == EINTR) ? Idle : IoError;
    buf_.append(chunk, static_cast<size_t>(n));
    return take_line(line) ? Line : Idle;
  }

  // SIGKILL (a masked SIGTERM could leave waitpid hanging), reap, close.
  void kill_and_reap() {
    if (pid_ > 0) {
      ::kill(-pid_, SIGKILL);
      ::kill(pid_, SIGKILL);
      int st = 0;
      while (waitpid(pid_, &st, 0) < 0 && errno == EINTR) {}
      exit_status_ = st;
      pid_ = -1;
    }
    if (fd_ >= 0) { close(fd_); fd_ = -1; }
    peer_open_ = false;
  }
  int exit_status() const { return exit_status_; }

 private:
  bool take_line(std::string* line) {
    size_t nl = buf_.find('\n');
    if (nl == std::string::npos) return false;
    *line = buf_.substr(0, nl);
    buf_.erase(0, nl + 1);
    return true;
  }
  int fd_ = -1;
  pid_t pid_ = -1;
  bool peer_open_ = false;
  int exit_status_ = 0;
  std::string buf_;
};

}  // namespace mdb
