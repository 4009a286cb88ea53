#include "utils/rendezvous.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>
#include <vector>

namespace hetuCTR {

namespace {

using Clock = std::chrono::steady_clock;

double since(Clock::time_point t0) { return std::chrono::duration<double>(Clock::now() - t0).count(); }

void fail(const std::string &what) { throw std::runtime_error("TCPRendezvous: " + what); }

// Full-length send/recv with a deadline; the sockets are blocking, poll() bounds each wait.
void io_all(int fd, void *buf, size_t len, bool sending, Clock::time_point t0, double timeout_s) {
  char *p = static_cast<char *>(buf);
  while (len > 0) {
    double left = timeout_s - since(t0);
    if (left <= 0) fail("timed out during transfer");
    pollfd pf{fd, static_cast<short>(sending ? POLLOUT : POLLIN), 0};
    int pr = poll(&pf, 1, (int)(left * 1000) + 1);
    if (pr < 0 && errno == EINTR) continue;
    if (pr <= 0) fail("timed out during transfer");
    ssize_t n = sending ? ::send(fd, p, len, MSG_NOSIGNAL) : ::recv(fd, p, len, 0);
    if (n < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (n <= 0) fail(std::string("peer closed the connection: ") + std::strerror(errno));
    p += n;
    len -= (size_t)n;
  }
}

sockaddr_in make_addr(const std::string &ip, int port) {
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)port);
  if (inet_pton(AF_INET, ip.c_str(), &a.sin_addr) != 1) fail("not an IPv4 address: " + ip);
  return a;
}

}  // namespace

TCPRendezvous::TCPRendezvous(int rank, int nrank, std::string ip, int port, double timeout_s)
    : rank_(rank), nrank_(nrank), port_(port), ip_(std::move(ip)), timeout_s_(timeout_s) {
  if (rank < 0 || rank >= nrank) fail("rank out of range");
}

void TCPRendezvous::broadcast(void *data, size_t len) {
  if (nrank_ <= 1) return;
  const auto t0 = Clock::now();
  if (rank_ == 0) {
    int ls = ::socket(AF_INET, SOCK_STREAM, 0);
    if (ls < 0) fail("socket() failed");
    int one = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a = make_addr(ip_, port_);
    if (::bind(ls, reinterpret_cast<sockaddr *>(&a), sizeof(a)) != 0) {
      ::close(ls);
      fail("cannot bind " + ip_ + ":" + std::to_string(port_) + ": " + std::strerror(errno));
    }
    ::listen(ls, nrank_);
    std::vector<int> peers;
    std::vector<bool> seen(nrank_, false);
    try {
      while ((int)peers.size() < nrank_ - 1) {
        double left = timeout_s_ - since(t0);
        if (left <= 0) fail("only " + std::to_string(peers.size() + 1) + " of " + std::to_string(nrank_) + " ranks arrived");
        pollfd pf{ls, POLLIN, 0};
        int pr = poll(&pf, 1, (int)(left * 1000) + 1);
        if (pr < 0 && errno == EINTR) continue;
        if (pr <= 0) continue;
        int fd = ::accept(ls, nullptr, nullptr);
        if (fd < 0) continue;
        peers.push_back(fd);
        int32_t who = -1;
        io_all(fd, &who, sizeof(who), false, t0, timeout_s_);
        if (who <= 0 || who >= nrank_ || seen[who]) fail("unexpected rank id " + std::to_string(who));
        seen[who] = true;
      }
      for (int fd : peers) io_all(fd, data, len, true, t0, timeout_s_);
      // wait for each peer's acknowledgement so the listener outlives every transfer
      for (int fd : peers) {
        char ack = 0;
        io_all(fd, &ack, 1, false, t0, timeout_s_);
      }
    } catch (...) {
      for (int fd : peers) ::close(fd);
      ::close(ls);
      throw;
    }
    for (int fd : peers) ::close(fd);
    ::close(ls);
  } else {
    sockaddr_in a = make_addr(ip_, port_);
    int fd = -1;
    for (;;) {
      fd = ::socket(AF_INET, SOCK_STREAM, 0);
      if (fd < 0) fail("socket() failed");
      if (::connect(fd, reinterpret_cast<sockaddr *>(&a), sizeof(a)) == 0) break;
      ::close(fd);
      fd = -1;
      if (since(t0) > timeout_s_) fail("rank 0 not reachable at " + ip_ + ":" + std::to_string(port_));
      std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    try {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      int32_t who = rank_;
      io_all(fd, &who, sizeof(who), true, t0, timeout_s_);
      io_all(fd, data, len, false, t0, timeout_s_);
      char ack = 1;
      io_all(fd, &ack, 1, true, t0, timeout_s_);
    } catch (...) {
      ::close(fd);
      throw;
    }
    ::close(fd);
  }
}

}  // namespace hetuCTR
