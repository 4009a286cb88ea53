// TEST INFRASTRUCTURE.  Stand-in for the reference's utils/rendezvous.h, which needs <zmq.h> (not present
// in this image).  Placed ahead of the reference's csrc on the include path when oracle/_ref is built: the
// reference's table_initialize.cu only constructs TCPRendezvous(rank, nrank, ip, port) and calls
// broadcast(ptr, len), both of which this repository's POSIX-socket implementation provides.
#pragma once
#include "../../../hetuctr_b200/csrc/utils/rendezvous.h"
