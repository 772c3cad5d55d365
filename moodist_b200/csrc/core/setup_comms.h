// Bootstrap ring: before any data plane exists, every rank can reach every other one through a ring of
// TCP connections built from nothing but a key/value store.
//
// Each rank listens on an ephemeral port, publishes its addresses through the store, and connects to the
// next rank only; a message for any other rank is forwarded around the ring with a TTL. Frame body:
//     u64 sig | u64 senderId | u32 src | u32 dst | u32 ttl | payload
// sig = 0x116dc74103a4dc0f for routed messages, 0x116dc74102a4dc0f for the ring all-gather; the first frame
// on a connection has dst = ~0 and payload "connect" + groupKey (reference: core/setup_comms.cc:12-13,
// 128-146, 257-314; core/setup_comms.h:45-67). Typed helpers prefix the payload with a type name so a
// receiver that expects another type fails loudly instead of misreading bytes.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <typeinfo>
#include <vector>

#include "kvstore.h"
#include "wire.h"

namespace moodist {

constexpr uint64_t kSetupSigMessage = 0x116dc74103a4dc0full;
constexpr uint64_t kSetupSigAllGather = 0x116dc74102a4dc0full;

class SetupComms {
 public:
  static std::unique_ptr<SetupComms> create(KVStore& store, const std::string& group_key, int rank, int world,
                                            double timeout_s = 60.0);
  virtual ~SetupComms() = default;

  // Every rank contributes one blob; returns all of them indexed by rank. Collective.
  virtual std::vector<Bytes> allgather_bytes(const Bytes& mine) = 0;
  // Point to point through the ring (blocking receive with the constructor's timeout).
  virtual void send_bytes(int dst, const Bytes& payload) = 0;
  virtual Bytes recv_bytes(int src) = 0;

  template <class T>
  std::vector<T> allgather(const T& v) {
    std::vector<Bytes> all = allgather_bytes(encode(std::string(typeid(T).name()), v));
    std::vector<T> out(all.size());
    for (size_t i = 0; i < all.size(); ++i) {
      std::string tn;
      Reader r(all[i]);
      r(tn);
      if (tn != typeid(T).name()) throw WireError("setup comms: all-gather type mismatch (" + tn + ")");
      r(out[i]);
    }
    return out;
  }
  template <class T>
  void send_to(int dst, const T& v) {
    send_bytes(dst, encode(std::string(typeid(T).name()), v));
  }
  template <class T>
  T recv_from(int src) {
    Bytes b = recv_bytes(src);
    std::string tn;
    T v{};
    Reader r(b);
    r(tn);
    if (tn != typeid(T).name()) throw WireError("setup comms: expected " + std::string(typeid(T).name()) + ", got " + tn);
    r(v);
    return v;
  }
};

}  // namespace moodist
