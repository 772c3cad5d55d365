// Minimal key/value rendezvous interface the core needs from "a store". Implemented by the library's
// own TcpStore and by an adapter over any c10d::Store in the torch glue, so the core stays torch-free
// (the reference reaches c10d stores through function pointers in its WrapperApi table,
// api/moodist_api.h:61-129).
#pragma once

#include <chrono>
#include <cstdint>
#include <string>
#include <vector>

namespace moodist {

class KVStore {
 public:
  virtual ~KVStore() = default;
  virtual void set(const std::string& key, const std::vector<uint8_t>& value) = 0;
  // Blocks until the key exists (or the store's timeout expires: throws).
  virtual std::vector<uint8_t> get(const std::string& key) = 0;
  virtual bool check(const std::vector<std::string>& keys) = 0;
  virtual void wait(const std::vector<std::string>& keys) = 0;

  void set_str(const std::string& key, const std::string& v) { set(key, std::vector<uint8_t>(v.begin(), v.end())); }
  std::string get_str(const std::string& key) {
    auto b = get(key);
    return std::string(b.begin(), b.end());
  }
  // All ranks call with the same tag; returns when everyone has.
  void barrier(const std::string& tag, int rank, int world) {
    set_str(tag + "/" + std::to_string(rank), "1");
    for (int r = 0; r < world; ++r) get(tag + "/" + std::to_string(r));
  }
};

}  // namespace moodist
