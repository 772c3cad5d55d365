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
};

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

  uint64_t bytes_sent() const { return bytes_sent_; }
  uint64_t bytes_received() const { return bytes_recv_; }

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
  };
  std::unordered_map<uint64_t, Pending> pending_;
  uint64_t bytes_sent_ = 0, bytes_recv_ = 0;
  Bytes sink_;
};

}  // namespace moodist
