// Binary wire format used by every control-plane message of the library (store, bootstrap ring,
// transport greetings, engine messages, queue records).
//
// Format (byte-compatible with the reference's serializer, core/serialization.h:77-250, 496-635):
//   * native little-endian, no padding between fields, no type tags;
//   * trivially copyable T            -> sizeof(T) raw bytes;
//   * string / string_view            -> u64 length + bytes;
//   * vector<T>                       -> u64 count + elements;
//   * map / unordered_map             -> u64 count + (key, value)...;
//   * optional<T>                     -> u8 has_value + value;
//   * variant<Ts...>                  -> u64 index + value;
//   * pair / tuple                    -> fields in order;
//   * user types                      -> whatever their `template <class Ar> void wire(Ar&)` visits.
// Reading past the end or leaving trailing bytes (decode_exact) throws WireError.
//
// The implementation is written around two archive classes (Writer, Reader) and C++20 concepts rather
// than the reference's SFINAE operator() chain.
#pragma once

#include <concepts>
#include <cstdint>
#include <cstring>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <string_view>
#include <tuple>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <variant>
#include <vector>

namespace moodist {

struct WireError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

using Bytes = std::vector<uint8_t>;

class Writer;
class Reader;

template <class T>
concept HasWire = requires(T& t, Writer& w) { t.wire(w); };

template <class T>
concept RawCopyable = std::is_trivially_copyable_v<T> && !HasWire<T> && !std::is_pointer_v<T>;

template <class T>
struct is_std_vector : std::false_type {};
template <class T, class A>
struct is_std_vector<std::vector<T, A>> : std::true_type {};
template <class T>
struct is_std_map : std::false_type {};
template <class K, class V, class C, class A>
struct is_std_map<std::map<K, V, C, A>> : std::true_type {};
template <class K, class V, class H, class E, class A>
struct is_std_map<std::unordered_map<K, V, H, E, A>> : std::true_type {};
template <class T>
struct is_std_optional : std::false_type {};
template <class T>
struct is_std_optional<std::optional<T>> : std::true_type {};
template <class T>
struct is_std_variant : std::false_type {};
template <class... T>
struct is_std_variant<std::variant<T...>> : std::true_type {};
template <class T>
struct is_std_pair : std::false_type {};
template <class A, class B>
struct is_std_pair<std::pair<A, B>> : std::true_type {};
template <class T>
struct is_std_tuple : std::false_type {};
template <class... T>
struct is_std_tuple<std::tuple<T...>> : std::true_type {};

class Writer {
 public:
  static constexpr bool kReading = false;
  Bytes out;

  void raw(const void* p, size_t n) {
    if (n == 0) return;  // p may be null then
    const uint8_t* b = static_cast<const uint8_t*>(p);
    out.insert(out.end(), b, b + n);
  }
  // overwrite previously written bytes (used to patch sequence numbers in place)
  void patch(size_t at, const void* p, size_t n) { std::memcpy(out.data() + at, p, n); }

  template <class... T>
  Writer& operator()(const T&... v) {
    (put(v), ...);
    return *this;
  }

  template <class T>
  void put(const T& v) {
    using U = std::remove_cvref_t<T>;
    if constexpr (std::is_same_v<U, std::string> || std::is_same_v<U, std::string_view>) {
      uint64_t n = v.size();
      raw(&n, 8);
      raw(v.data(), n);
    } else if constexpr (std::is_convertible_v<U, const char*>) {
      put(std::string_view(v));
    } else if constexpr (is_std_vector<U>::value) {
      uint64_t n = v.size();
      raw(&n, 8);
      using E = typename U::value_type;
      if constexpr (RawCopyable<E> && !std::is_same_v<E, bool>) {
        raw(v.data(), n * sizeof(E));
      } else {
        for (const auto& e : v) put(e);
      }
    } else if constexpr (is_std_map<U>::value) {
      uint64_t n = v.size();
      raw(&n, 8);
      for (const auto& [k, e] : v) {
        put(k);
        put(e);
      }
    } else if constexpr (is_std_optional<U>::value) {
      uint8_t has = v.has_value();
      raw(&has, 1);
      if (has) put(*v);
    } else if constexpr (is_std_variant<U>::value) {
      uint64_t idx = v.index();
      raw(&idx, 8);
      std::visit([&](const auto& e) { put(e); }, v);
    } else if constexpr (is_std_pair<U>::value) {
      put(v.first);
      put(v.second);
    } else if constexpr (is_std_tuple<U>::value) {
      std::apply([&](const auto&... e) { (put(e), ...); }, v);
    } else if constexpr (HasWire<U>) {
      const_cast<U&>(v).wire(*this);
    } else {
      static_assert(RawCopyable<U>, "type has no wire format");
      raw(&v, sizeof(U));
    }
  }
};

class Reader {
 public:
  static constexpr bool kReading = true;
  const uint8_t* p;
  const uint8_t* end;

  Reader(const void* data, size_t n) : p(static_cast<const uint8_t*>(data)), end(p + n) {}
  explicit Reader(const Bytes& b) : Reader(b.data(), b.size()) {}

  size_t remaining() const { return static_cast<size_t>(end - p); }
  const uint8_t* take(size_t n) {
    if (n > remaining()) throw WireError("wire: read past end of message");
    const uint8_t* r = p;
    p += n;
    return r;
  }
  void raw(void* dst, size_t n) {
    const uint8_t* src = take(n);
    if (n) std::memcpy(dst, src, n);  // an empty vector's data() may be null, which memcpy must not be given
  }

  template <class... T>
  Reader& operator()(T&... v) {
    (get(v), ...);
    return *this;
  }
  template <class T>
  T read() {
    T v{};
    get(v);
    return v;
  }
  std::string_view view() {
    uint64_t n;
    raw(&n, 8);
    const uint8_t* b = take(n);
    return {reinterpret_cast<const char*>(b), static_cast<size_t>(n)};
  }

  template <class T>
  void get(T& v) {
    using U = std::remove_cvref_t<T>;
    if constexpr (std::is_same_v<U, std::string>) {
      v = std::string(view());
    } else if constexpr (std::is_same_v<U, std::string_view>) {
      v = view();
    } else if constexpr (is_std_vector<U>::value) {
      uint64_t n;
      raw(&n, 8);
      using E = typename U::value_type;
      if constexpr (RawCopyable<E> && !std::is_same_v<E, bool>) {
        if (n > remaining() / sizeof(E)) throw WireError("wire: vector length exceeds message");
        v.resize(n);
        raw(v.data(), n * sizeof(E));
      } else {
        if (n > remaining()) throw WireError("wire: vector length exceeds message");
        v.clear();
        v.reserve(n);
        for (uint64_t i = 0; i < n; ++i) {
          E e{};
          get(e);
          v.push_back(std::move(e));
        }
      }
    } else if constexpr (is_std_map<U>::value) {
      uint64_t n;
      raw(&n, 8);
      if (n > remaining()) throw WireError("wire: map length exceeds message");
      v.clear();
      for (uint64_t i = 0; i < n; ++i) {
        typename U::key_type k{};
        typename U::mapped_type e{};
        get(k);
        get(e);
        v.emplace(std::move(k), std::move(e));
      }
    } else if constexpr (is_std_optional<U>::value) {
      uint8_t has;
      raw(&has, 1);
      if (has) {
        v.emplace();
        get(*v);
      } else {
        v.reset();
      }
    } else if constexpr (is_std_variant<U>::value) {
      uint64_t idx;
      raw(&idx, 8);
      if (idx >= std::variant_size_v<U>) throw WireError("wire: bad variant index");
      emplace_variant<0>(v, idx);
    } else if constexpr (is_std_pair<U>::value) {
      get(v.first);
      get(v.second);
    } else if constexpr (is_std_tuple<U>::value) {
      std::apply([&](auto&... e) { (get(e), ...); }, v);
    } else if constexpr (HasWire<U>) {
      v.wire(*this);
    } else {
      static_assert(RawCopyable<U>, "type has no wire format");
      raw(&v, sizeof(U));
    }
  }

 private:
  template <size_t I, class V>
  void emplace_variant(V& v, uint64_t idx) {
    if constexpr (I < std::variant_size_v<V>) {
      if (idx == I) {
        get(v.template emplace<I>());
      } else {
        emplace_variant<I + 1>(v, idx);
      }
    }
  }
};

template <class... T>
Bytes encode(const T&... v) {
  Writer w;
  w(v...);
  return std::move(w.out);
}

// decode and require that the whole buffer was consumed
template <class... T>
void decode_exact(const void* data, size_t n, T&... v) {
  Reader r(data, n);
  r(v...);
  if (r.remaining() != 0) throw WireError("wire: " + std::to_string(r.remaining()) + " trailing bytes");
}
template <class... T>
void decode_exact(const Bytes& b, T&... v) {
  decode_exact(b.data(), b.size(), v...);
}
// decode a prefix; returns the number of bytes consumed
template <class... T>
size_t decode_prefix(const void* data, size_t n, T&... v) {
  Reader r(data, n);
  r(v...);
  return n - r.remaining();
}

inline std::string to_hex(const Bytes& b) {
  static const char* d = "0123456789abcdef";
  std::string s;
  s.reserve(b.size() * 2);
  for (uint8_t c : b) {
    s.push_back(d[c >> 4]);
    s.push_back(d[c & 15]);
  }
  return s;
}
inline Bytes from_hex(std::string_view s) {
  auto nib = [](char c) -> int {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    if (c >= 'A' && c <= 'F') return c - 'A' + 10;
    throw WireError("wire: bad hex digit");
  };
  if (s.size() % 2) throw WireError("wire: odd hex length");
  Bytes b(s.size() / 2);
  for (size_t i = 0; i < b.size(); ++i) b[i] = static_cast<uint8_t>(nib(s[2 * i]) << 4 | nib(s[2 * i + 1]));
  return b;
}

}  // namespace moodist
