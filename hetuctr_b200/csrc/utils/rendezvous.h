// Bootstrap broadcast over plain TCP: rank 0 listens on (ip, port) and sends a small blob (the NCCL
// unique id) to every other rank.  Same role and constructor arguments as the reference's
// TCPRendezvous (csrc/utils/rendezvous.h:14-45), but over POSIX sockets with deadlines instead of
// blocking forever.
#pragma once
#include <cstddef>
#include <string>

namespace hetuCTR {

class TCPRendezvous {
 public:
  TCPRendezvous(int rank, int nrank, std::string ip, int port, double timeout_s = 120.0);
  // Copies `len` bytes at `data` from rank 0 to all ranks.  Throws std::runtime_error on timeout.
  void broadcast(void *data, size_t len);

 private:
  int rank_, nrank_, port_;
  std::string ip_;
  double timeout_s_;
};

}  // namespace hetuCTR
