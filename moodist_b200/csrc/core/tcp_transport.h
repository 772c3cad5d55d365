// TCP data plane: a full mesh of connections between the ranks of a group carrying an emulation of
// one-sided RDMA (write / read against registered memory regions) plus two-sided sends.
//
// Wire behaviour follows the reference's TcpDev + RdmaTcp (core/tcpdev.cc:15, 92-106, 187-219;
// core/rdma_tcp.cc:9-99, 106-525):
//   * the lower rank dials every higher rank at all of its advertised addresses; the first connection
//     that completes the greeting  u64 0x5a59123966da2598 | string groupName | u32 rank  is kept;
//   * message types (u8): Write 1, CompletionSuccess 2, CompletionError 3, Send 4, Read 5, ReadSuccess 6;
//   * lkey/rkey are indices into a process-global table of registered regions, every remote access is
//     bounds-checked against it, and payloads are read from the socket straight into the destination;
//   * sends issued before the connection exists are queued.
// Each record header travels as one frame (net.h); Write / Send / ReadSuccess payload bytes follow the
// frame on the stream.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "net.h"

namespace moodist {

constexpr uint64_t kTcpDevSig = 0x5a59123966da2598ull;

enum TcpMsg : uint8_t {
  kMsgWrite = 1,
  kMsgCompletionSuccess = 2,
  kMsgCompletionError = 3,
  kMsgSend = 4,
  kMsgRead = 5,
  kMsgReadSuccess = 6,
  // extension (not in the reference's record set): one request for `rows` runs of `row_bytes` bytes that lie
  // `src_pitch` apart; answered by one ReadSuccess whose payload is the runs back to back
  kMsgReadStrided = 7,
  // extensions for two ranks on one machine that may read each other's address space (process_vm_readv):
  // the bytes move with one copy made by the process that receives them, the connection only carries the
  // request, the owner's bounds check and the completion.
  kMsgDirectOk = 8,     // u8 | i64 pid : "I can read your memory" (sent once, after a successful probe)
  kMsgWriteDirect = 9,  // u8 | u64 index | u32 rkey | uptr raddr | size_t bytes | uptr source address
  kMsgReadCheck = 10,   // u8 | u64 index | u32 rkey | uptr raddr | size_t span : owner answers Granted / Error
  kMsgReadGranted = 11, // u8 | u64 index
};

// Copies between this process and `pid` with process_vm_readv (the reference moves CPU tensors between ranks
// of one machine the same way, core/cputhread.cc:3369-3379). False when the kernel refuses (ptrace rules,
// another PID namespace) or the copy comes up short.
bool vm_read(int64_t pid, void* local, uintptr_t remote, size_t bytes);
bool vm_read_strided(int64_t pid, void* local, size_t dst_pitch, uintptr_t remote, size_t src_pitch, uint64_t rows,
                     size_t row_bytes);

// Process-global registered-memory table (reference: MrManager, core/rdma_tcp.cc:17-65).
class MrTable {
 public:
  static MrTable& instance();
  uint32_t add(void* base, size_t size);
  void remove(uint32_t key);
  // Returns the address if [addr, addr+bytes) lies inside region `key`, else nullptr.
  void* check(uint32_t key, uintptr_t addr, size_t bytes);
  // Bytes written into the region by remote writes so far.
  uint64_t landed(uint32_t key);
  void add_landed(uint32_t key, uint64_t n);
};

class TcpTransport {
 public:
  using Done = std::function<void(bool ok)>;
  using RecvFn = std::function<void(int src, Bytes payload)>;
  using ErrorFn = std::function<void(int peer, const std::string& why)>;

  TcpTransport(Poller& poller, std::string group, int rank, int world);
  ~TcpTransport();

  // Open listeners; returns the "host port" strings other ranks can dial.
  std::vector<std::string> listen();
  // addrs[r] = what rank r's listen() returned. Dials the higher ranks.
  void connect_all(const std::vector<std::vector<std::string>>& addrs);
  bool all_connected() const;
  // Between hold_sends() and release_sends() records only queue on their connections; release_sends() writes each
  // connection's backlog with as few system calls as it takes. For a caller about to send a burst.
  // how many peers are reached over a unix-domain socket (same machine, same network namespace)
  int unix_peers() const;
  void hold_sends();
  void release_sends();
  int connected_count() const;

  void on_recv(RecvFn f) { recv_ = std::move(f); }
  void on_error(ErrorFn f) { error_ = std::move(f); }

  // One-sided write of local memory into a peer's registered region. `keep` pins the source.
  void post_write(int dst, const void* src, size_t bytes, uint32_t rkey, uintptr_t raddr, Done done,
                  std::shared_ptr<void> keep = nullptr);
  // One-sided read of a peer's registered region into local memory.
  void post_read(int dst, void* local, size_t bytes, uint32_t rkey, uintptr_t raddr, Done done);
  // rows x row_bytes from raddr + r * src_pitch into local + r * dst_pitch, one request and one reply
  void post_read_strided(int dst, void* local, uint64_t rows, size_t row_bytes, size_t dst_pitch, uint32_t rkey,
                         uintptr_t raddr, size_t src_pitch, Done done);
  // Two-sided message.
  void post_send(int dst, Bytes payload);

  // Test hook: drop / delay / duplicate outgoing two-sided messages (host-side fault injection).
  // Return 0 to send normally, 1 to drop, 2 to send twice.
  std::function<int(int dst, const Bytes& payload)> fault_hook;

  // Same-machine fast path. probe_direct: try to read the 8-byte word at `probe_addr` of process `pid` (rank
  // `peer`); when it holds `probe_value` this rank may read that process, remembers it and tells the peer,
  // which from then on lets this rank fetch the payload of its writes itself. Transfers below
  // `direct_min_bytes` keep travelling inline on the connection.
  bool probe_direct(int peer, int64_t pid, uintptr_t probe_addr, uint64_t probe_value);
  void set_direct_min_bytes(size_t n) { direct_min_ = n; }

  uint64_t bytes_sent() const { return bytes_sent_; }
  uint64_t bytes_received() const { return bytes_recv_; }
  uint64_t bytes_direct() const { return bytes_direct_; }  // payload bytes copied with process_vm_readv

 private:
  struct Peer;
  void attach(int peer, std::shared_ptr<Conn> c);
  void handle_record(int peer, Reader& r);
  void send_record(int peer, Bytes header, const void* payload, size_t n, std::shared_ptr<void> keep);
  void deliver_local(std::function<void()> fn);

  Poller& poller_;
  std::string group_;
  int rank_, world_;
  std::vector<std::unique_ptr<Peer>> peers_;
  RecvFn recv_;
  ErrorFn error_;
  uint64_t next_index_ = 1;
  struct Pending {
    Done done;
    void* local = nullptr;
    size_t bytes = 0;
    uint64_t rows = 1;        // > 1: the reply is scattered, row_bytes at a time, dst_pitch apart
    size_t row_bytes = 0, dst_pitch = 0;
    std::shared_ptr<void> keep;  // direct writes: the source stays alive until the receiver has fetched it
    uintptr_t raddr = 0;         // direct reads: what to fetch once the owner has granted it
    size_t src_pitch = 0;
    int peer = -1;
  };
  std::unordered_map<uint64_t, Pending> pending_;
  uint64_t bytes_sent_ = 0, bytes_recv_ = 0, bytes_direct_ = 0;
  size_t direct_min_ = 8192;
  Bytes sink_;
};

}  // namespace moodist
