// TcpStore: a decentralised key/value store used for rendezvous (moodist.TcpStore).
//
// Behaviour follows the reference's StoreImpl (core/store.cc, docs/internals/tcp_store.md):
//   * every key has an owner rank, owner = stringHash(key) % world with the same hash function
//     (core/store.cc:1733-1743), so no single rank serves all traffic;
//   * ranks form a sparse mesh — a ring for world <= 4, ring plus one pseudo-random chord per rank
//     otherwise, at most 4 edges per rank, seeded by the store identity so every rank computes the same
//     graph (core/store.cc:1146-1251) — and requests are forwarded along BFS first-hop routes with a TTL;
//   * every edge numbers its messages, acknowledges them and retransmits what was not acknowledged after
//     a reconnect; idle edges exchange keepalives (core/store.cc:1563-1615, 2015-2054);
//   * message types on the wire: Done 3, Set 4, Get 5, Check 6, Wait 7, Shutdown 8, Exit 9, ExitAck 10
//     (core/store.cc:31-39) inside `u64 0x220a74d1a52672b8 | MessageHeader | payload` frames;
//   * shutdown is three-phase (Shutdown, Exit, ExitAck) so a coordinated exit of all ranks raises no
//     error, while a rank that leaves alone makes the others' pending and later operations fail with
//     "store was shut down on rank X" (core/store.cc:1477-1548, 2115-2125);
//   * blocking calls wake once a second and fail after `timeout` with a message that says which hop
//     of the route is not answering.
// Differences, on purpose: the first contact with rank 0 uses a TCP connection to hostname:port instead
// of UDP datagrams (works on loopback and through firewalls that drop UDP), and add / compare_set /
// delete_key / num_keys are implemented instead of throwing.
#pragma once

#include <chrono>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "kvstore.h"

namespace moodist {

uint32_t store_string_hash(const std::string& s);

class TcpStore : public KVStore {
 public:
  static std::shared_ptr<TcpStore> create(const std::string& hostname, int port, const std::string& key, int world,
                                          int rank, std::chrono::milliseconds timeout);
  ~TcpStore() override = default;

  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual std::chrono::milliseconds timeout() const = 0;
  virtual void set_timeout(std::chrono::milliseconds t) = 0;

  // KVStore: set / get / check / wait(keys)
  virtual void wait_for(const std::vector<std::string>& keys, std::chrono::milliseconds timeout) = 0;
  virtual int64_t add(const std::string& key, int64_t delta) = 0;
  virtual std::vector<uint8_t> compare_set(const std::string& key, const std::vector<uint8_t>& expected,
                                           const std::vector<uint8_t>& desired) = 0;
  virtual bool delete_key(const std::string& key) = 0;
  virtual int64_t num_keys() = 0;

  // Starts the coordinated shutdown; called by the destructor of the last handle.
  virtual void shutdown() = 0;
  // Coordinated shutdown of every store of this process that is still alive. For the end of a process whose store
  // objects were never destroyed (kept by a reference cycle, a global): a rank that just vanishes takes the answers
  // it had queued for its peers with it.
  static void shutdown_all();

  // Host-side fault injection for tests: from now on every `break_every`-th message this rank sends over a mesh
  // edge is lost together with its connection (0 switches it off). The edge redials and retransmits.
  virtual void inject_faults(int break_every) = 0;
  virtual uint64_t injected_breaks() = 0;

  // Mesh introspection (tests, diagnostics)
  virtual std::vector<int> edges() const = 0;
  virtual std::string describe() const = 0;
};

// The mesh every rank computes for (world, seed): adjacency lists, <= 4 edges per rank, connected.
std::vector<std::vector<int>> store_mesh(int world, uint32_t seed);
// first_hop[dst] for `rank` on that mesh (BFS).
std::vector<int> store_first_hops(const std::vector<std::vector<int>>& mesh, int rank);

}  // namespace moodist
