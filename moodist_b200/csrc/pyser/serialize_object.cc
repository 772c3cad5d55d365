// Python-object serializer (module `moodist_b200._serialize`): a faster, more compact pickle
// replacement used by Queue.put_object / get_object and compile_op's metadata exchange.
//
// Byte format (identical to the reference, wrapper/serialize/serialize_object.cc:36-58, 293-337,
// 524-556, 582-591, 651-748, 827-836, 854-859):
//   every value starts with a one-byte tag
//     0 none | 1 True | 2 False | 3 int8 | 4 int16 | 5 int32 | 6 int64 | 7 float (8-byte double)
//     8 dict | 9 str (legacy, never written) | 10 list | 11 tuple | 12 bigint | 13 unicode | 14 bytes
//     15 bytearray | 16 set | 17 frozenset | 18 global | 19 class | 20 offset
//   ints use the smallest of 1/2/4/8 little-endian bytes; ints that are not "compact" in CPython
//   (|v| >= 2^30) are written as bigint: u64 byte count + two's-complement little-endian bytes
//   ((bits+7)/8 + 1 of them);
//   list / tuple / dict carry their length as an int value (tag + bytes); set / frozenset as a raw u64;
//   unicode = u8 kind (1, 2 or 4) + u64 byte count + raw UCS1/2/4 code units;
//   bytes / bytearray = u64 count + bytes;
//   global = qualified name value + module name value (functions and classes);
//   class = callable value + args value + u8 bits {1 state, 2 list items, 4 dict items, 8 setstate} +
//           [state [setstate]] [list value] [u64 n + n (key, value) pairs]   (from __reduce_ex__(5));
//   shared and circular references: every container / string / object remembers the offset of its tag
//   byte; when the same object is met again the ORIGINAL tag byte gets bit 0x80 set and an
//   `offset` record (tag 20 + u64 offset) is written instead. A reader stores every value whose tag
//   has 0x80 set under its offset before reading its children.
//
// Written against the CPython C API only (no pybind11), with explicit Packer / Unpacker classes.
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <cstdint>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

enum Tag : uint8_t {
  T_NONE = 0,
  T_TRUE = 1,
  T_FALSE = 2,
  T_INT8 = 3,
  T_INT16 = 4,
  T_INT32 = 5,
  T_INT64 = 6,
  T_FLOAT = 7,
  T_DICT = 8,
  T_STR = 9,
  T_LIST = 10,
  T_TUPLE = 11,
  T_BIGINT = 12,
  T_UNICODE = 13,
  T_BYTES = 14,
  T_BYTEARRAY = 15,
  T_SET = 16,
  T_FROZENSET = 17,
  T_GLOBAL = 18,
  T_CLASS = 19,
  T_OFFSET = 20,
};

struct PyError {};  // a Python exception is already set

struct Ref {  // owning reference
  PyObject* p = nullptr;
  Ref() = default;
  explicit Ref(PyObject* o) : p(o) {}
  Ref(const Ref&) = delete;
  Ref& operator=(const Ref&) = delete;
  Ref(Ref&& o) noexcept : p(o.p) { o.p = nullptr; }
  Ref& operator=(Ref&& o) noexcept {
    std::swap(p, o.p);
    return *this;
  }
  ~Ref() { Py_XDECREF(p); }
  PyObject* release() {
    PyObject* r = p;
    p = nullptr;
    return r;
  }
  explicit operator bool() const { return p != nullptr; }
};

Ref checked(PyObject* o) {
  if (!o) throw PyError{};
  return Ref(o);
}

PyObject *s_qualname, *s_module, *s_reduce_ex, *s_dict, *s_setstate, *s_dot, *s_extend, *s_append, *s_five;
PyObject* g_dispatch_table;  // copyreg.dispatch_table: type -> reducer
PyObject* g_newobj;  // copyreg.__newobj__, what object.__reduce_ex__(2+) names as the constructor

void init_strings() {
  if (s_qualname) return;
  s_qualname = PyUnicode_InternFromString("__qualname__");
  s_module = PyUnicode_InternFromString("__module__");
  s_reduce_ex = PyUnicode_InternFromString("__reduce_ex__");
  s_dict = PyUnicode_InternFromString("__dict__");
  s_setstate = PyUnicode_InternFromString("__setstate__");
  s_dot = PyUnicode_InternFromString(".");
  s_extend = PyUnicode_InternFromString("extend");
  s_append = PyUnicode_InternFromString("append");
  s_five = PyLong_FromLong(5);
  if (PyObject* copyreg = PyImport_ImportModule("copyreg")) {
    g_newobj = PyObject_GetAttrString(copyreg, "__newobj__");
    g_dispatch_table = PyObject_GetAttrString(copyreg, "dispatch_table");
    if (g_dispatch_table && !PyDict_Check(g_dispatch_table)) Py_CLEAR(g_dispatch_table);
    Py_DECREF(copyreg);
  }
  if (!g_newobj || !g_dispatch_table) PyErr_Clear();
}

// ------------------------------------------------------------------------------------------------
// Output bytes: a growing buffer that lives in the bytearray the caller finally receives (no zero-fill on growth, no
// per-byte capacity check beyond one compare, no copy at the end).
class ByteBuf {
 public:
  ByteBuf() = default;
  ByteBuf(const ByteBuf&) = delete;
  ByteBuf& operator=(const ByteBuf&) = delete;
  ~ByteBuf() { Py_XDECREF(array_); }
  size_t size() const { return size_; }
  uint8_t* data() { return data_; }
  uint8_t& operator[](size_t i) { return data_[i]; }
  void reserve(size_t n) {
    if (n > cap_) grow(n);
  }
  void push_back(uint8_t b) {
    if (size_ == cap_) grow(size_ + 1);
    data_[size_++] = b;
  }
  void append(const void* p, size_t n) {
    if (size_ + n > cap_) grow(size_ + n);
    memcpy(data_ + size_, p, n);
    size_ += n;
  }
  // The bytes written so far as a bytearray (a new reference); the buffer is empty afterwards. The storage IS
  // the bytearray's, so nothing is copied however large the result.
  PyObject* release() {
    if (!array_) return PyByteArray_FromStringAndSize("", 0);
    if (PyByteArray_Resize(array_, (Py_ssize_t)size_) < 0) throw PyError{};
    PyObject* out = array_;
    array_ = nullptr;
    data_ = nullptr;
    size_ = cap_ = 0;
    return out;
  }

 private:
  // out of line and marked cold, so that push_back / append stay a compare, a store and an add where they are inlined
  __attribute__((noinline, cold)) void grow(size_t need) {
    size_t cap = cap_ ? cap_ * 2 : 256;
    if (cap < need) cap = need + (need >> 4);  // one large payload: no need to double past it
    if (!array_) {
      array_ = PyByteArray_FromStringAndSize(nullptr, (Py_ssize_t)cap);
      if (!array_) throw PyError{};
    } else if (PyByteArray_Resize(array_, (Py_ssize_t)cap) < 0) {
      throw PyError{};
    }
    data_ = reinterpret_cast<uint8_t*>(PyByteArray_AS_STRING(array_));
    cap_ = cap;
  }
  PyObject* array_ = nullptr;  // a bytearray whose storage is the buffer
  uint8_t* data_ = nullptr;
  size_t size_ = 0, cap_ = 0;
};

// Identity memo: object address -> offset of its first encoding. Open addressing with linear probing in a
// power-of-two table kept at most half full; one multiply to hash, no allocation per entry.
class PtrMap {
 public:
  PtrMap() { rehash(1024); }
  // returns {slot value reference, true if the key was inserted now}
  std::pair<size_t*, bool> try_emplace(PyObject* key, size_t value) {
    if ((count_ + 1) * 2 > keys_.size()) rehash(keys_.size() * 2);
    size_t i = index(key);
    while (keys_[i]) {
      if (keys_[i] == key) return {&vals_[i], false};
      i = (i + 1) & mask_;
    }
    keys_[i] = key;
    vals_[i] = value;
    ++count_;
    return {&vals_[i], true};
  }

 private:
  size_t index(PyObject* key) const {
    return (size_t)(((uint64_t)(uintptr_t)key >> 4) * 0x9E3779B97F4A7C15ull >> shift_);
  }
  void rehash(size_t n) {
    std::vector<PyObject*> ok;
    std::vector<size_t> ov;
    ok.swap(keys_);
    ov.swap(vals_);
    keys_.assign(n, nullptr);
    vals_.assign(n, 0);
    mask_ = n - 1;
    shift_ = 64 - __builtin_ctzll(n);
    count_ = 0;
    for (size_t j = 0; j < ok.size(); ++j)
      if (ok[j]) try_emplace(ok[j], ov[j]);
  }
  std::vector<PyObject*> keys_;
  std::vector<size_t> vals_;
  size_t mask_ = 0, count_ = 0;
  int shift_ = 0;
};

// Offsets of stored objects -> the objects, for the unpacker: open addressing on offset + 1 (0 marks an empty
// slot). Holds one reference per entry.
class OffsetMap {
 public:
  OffsetMap() { rehash(256); }
  ~OffsetMap() {
    for (size_t i = 0; i < keys_.size(); ++i)
      if (keys_[i]) Py_DECREF(vals_[i]);
  }
  OffsetMap(const OffsetMap&) = delete;
  OffsetMap& operator=(const OffsetMap&) = delete;

  PyObject* find(size_t offset) const {
    size_t key = offset + 1;
    for (size_t i = index(key); keys_[i]; i = (i + 1) & mask_)
      if (keys_[i] == key) return vals_[i];
    return nullptr;
  }
  // takes its own reference; a second object stored at the same offset replaces the first
  void put(size_t offset, PyObject* o) {
    if ((count_ + 1) * 2 > keys_.size()) rehash(keys_.size() * 2);
    Py_INCREF(o);
    size_t key = offset + 1;
    size_t i = index(key);
    for (; keys_[i]; i = (i + 1) & mask_) {
      if (keys_[i] == key) {
        Py_DECREF(vals_[i]);
        vals_[i] = o;
        return;
      }
    }
    keys_[i] = key;
    vals_[i] = o;
    ++count_;
  }

 private:
  size_t index(size_t key) const { return (size_t)((uint64_t)key * 0x9E3779B97F4A7C15ull >> shift_); }
  void rehash(size_t n) {
    std::vector<size_t> ok;
    std::vector<PyObject*> ov;
    ok.swap(keys_);
    ov.swap(vals_);
    keys_.assign(n, 0);
    vals_.assign(n, nullptr);
    mask_ = n - 1;
    shift_ = 64 - __builtin_ctzll(n);
    for (size_t j = 0; j < ok.size(); ++j) {
      if (!ok[j]) continue;
      size_t i = index(ok[j]);
      while (keys_[i]) i = (i + 1) & mask_;
      keys_[i] = ok[j];
      vals_[i] = ov[j];
    }
  }
  std::vector<size_t> keys_;
  std::vector<PyObject*> vals_;
  size_t mask_ = 0, count_ = 0;
  int shift_ = 0;
};

class Packer {
 public:
  ByteBuf out;

  void pack(PyObject* obj) {
    if (obj == Py_None) return byte(T_NONE);
    if (obj == Py_True) return byte(T_TRUE);
    if (obj == Py_False) return byte(T_FALSE);
    PyTypeObject* type = Py_TYPE(obj);
    if (type == &PyLong_Type) return pack_long(obj);
    if (type == &PyFloat_Type) {
      byte(T_FLOAT);
      double d = PyFloat_AS_DOUBLE(obj);
      raw(&d, 8);
      return;
    }
    // Everything below is memoised by identity, except objects with a single reference: whoever holds that
    // reference is the only way to reach them, so they cannot come up a second time (and cannot be the target of
    // a cycle, which would be a second reference). Skipping them keeps the memo small for the common case of
    // containers full of freshly built strings and tuples; the bytes produced are the same.
    if (Py_REFCNT(obj) != 1) {
      auto [slot, fresh] = memo_.try_emplace(obj, out.size());
      if (!fresh) {
        if (type == &PyFrozenSet_Type && std::find(open_frozensets_.begin(), open_frozensets_.end(), obj) != open_frozensets_.end()) {
          // it exists only once its members do, so a reader could not hand it to the member that wants it
          PyErr_SetString(PyExc_ValueError, "moodist.serialize: a frozenset that contains itself cannot be serialized");
          throw PyError{};
        }
        out[*slot] |= 0x80;
        byte(T_OFFSET);
        u64(*slot);
        return;
      }
    }
    if (depth_ > 2000) {
      PyErr_SetString(PyExc_RecursionError, "moodist.serialize: object nesting too deep");
      throw PyError{};
    }
    ++depth_;
    pack_object(obj, type);
    --depth_;
  }

 private:
  PtrMap memo_;
  std::vector<PyObject*> open_frozensets_;  // those whose members are being written
  std::vector<Ref> keepalive_;  // temporaries (reduce results) must outlive the memo entries that point at them
  int depth_ = 0;

  void byte(uint8_t b) { out.push_back(b); }
  void raw(const void* p, size_t n) { out.append(p, n); }
  void u64(uint64_t v) { raw(&v, 8); }

  void pack_int(int64_t v) {
    if (v == (int8_t)v) {
      byte(T_INT8);
      int8_t x = (int8_t)v;
      raw(&x, 1);
    } else if (v == (int16_t)v) {
      byte(T_INT16);
      int16_t x = (int16_t)v;
      raw(&x, 2);
    } else if (v == (int32_t)v) {
      byte(T_INT32);
      int32_t x = (int32_t)v;
      raw(&x, 4);
    } else {
      byte(T_INT64);
      raw(&v, 8);
    }
  }

  void pack_long(PyObject* obj) {
    if (PyUnstable_Long_IsCompact((PyLongObject*)obj)) return pack_int((int64_t)PyUnstable_Long_CompactValue((PyLongObject*)obj));
    size_t nbits = _PyLong_NumBits(obj);
    if (nbits == (size_t)-1 && PyErr_Occurred()) throw PyError{};
    size_t nbytes = (nbits + 7) / 8 + 1;
    std::vector<unsigned char> tmp(nbytes);
    if (_PyLong_AsByteArray((PyLongObject*)obj, tmp.data(), nbytes, 1, 1) < 0) throw PyError{};
    byte(T_BIGINT);
    u64(nbytes);
    raw(tmp.data(), nbytes);
  }

  void pack_items(uint8_t tag, PyObject** items, Py_ssize_t n) {
    byte(tag);
    pack_int(n);
    for (Py_ssize_t i = 0; i < n; ++i) pack(items[i]);
  }

  void pack_object(PyObject* obj, PyTypeObject* type) {
    if (type == &PyList_Type) {
      // the list may change size if a __reduce__ mutates it; index defensively
      byte(T_LIST);
      Py_ssize_t n = PyList_GET_SIZE(obj);
      pack_int(n);
      for (Py_ssize_t i = 0; i < n; ++i) {
        if (i >= PyList_GET_SIZE(obj)) {
          PyErr_SetString(PyExc_RuntimeError, "moodist.serialize: list changed size during serialization");
          throw PyError{};
        }
        pack(PyList_GET_ITEM(obj, i));
      }
      return;
    }
    if (type == &PyTuple_Type) return pack_items(T_TUPLE, &PyTuple_GET_ITEM(obj, 0), PyTuple_GET_SIZE(obj));
    if (type == &PyDict_Type) {
      byte(T_DICT);
      pack_int(PyDict_GET_SIZE(obj));
      Py_ssize_t pos = 0;
      PyObject *k, *v;
      while (PyDict_Next(obj, &pos, &k, &v)) {
        pack(k);
        pack(v);
      }
      return;
    }
    if (type == &PyUnicode_Type) {
      byte(T_UNICODE);
      uint8_t kind = (uint8_t)PyUnicode_KIND(obj);
      byte(kind);
      uint64_t nbytes = (uint64_t)PyUnicode_GET_LENGTH(obj) * kind;
      u64(nbytes);
      raw(PyUnicode_DATA(obj), nbytes);
      return;
    }
    if (type == &PyBytes_Type) {
      byte(T_BYTES);
      u64(PyBytes_GET_SIZE(obj));
      raw(PyBytes_AS_STRING(obj), PyBytes_GET_SIZE(obj));
      return;
    }
    if (type == &PyByteArray_Type) {
      byte(T_BYTEARRAY);
      u64(PyByteArray_GET_SIZE(obj));
      raw(PyByteArray_AS_STRING(obj), PyByteArray_GET_SIZE(obj));
      return;
    }
    if (type == &PySet_Type || type == &PyFrozenSet_Type) {
      byte(type == &PySet_Type ? T_SET : T_FROZENSET);
      u64(PySet_GET_SIZE(obj));
      if (type == &PyFrozenSet_Type) open_frozensets_.push_back(obj);
      Ref it = checked(PyObject_GetIter(obj));
      while (PyObject* item = PyIter_Next(it.p)) {
        Ref hold(item);
        pack(item);
      }
      if (PyErr_Occurred()) throw PyError{};
      if (type == &PyFrozenSet_Type) open_frozensets_.pop_back();
      return;
    }
    // classes of any metaclass are globals (the reference only recognises exact `type`, so e.g. numpy.dtype fails there)
    if (type == &PyFunction_Type || PyType_Check(obj)) return pack_global(obj);
    if (type == &PyPickleBuffer_Type) {
      // protocol-5 out-of-band buffers (numpy arrays reduce to these) are carried in-band, like pickle
      // does without a buffer_callback: writable -> bytearray, read-only -> bytes. The reference cannot
      // serialize these (tests/test_serialize.py:257-266).
      const Py_buffer* view = PyPickleBuffer_GetBuffer(obj);
      if (!view) throw PyError{};
      if (!PyBuffer_IsContiguous(view, 'A')) {
        PyErr_SetString(PyExc_ValueError, "moodist.serialize: cannot serialize a non-contiguous PickleBuffer");
        throw PyError{};
      }
      byte(view->readonly ? T_BYTES : T_BYTEARRAY);
      u64((uint64_t)view->len);
      raw(view->buf, (size_t)view->len);
      return;
    }
    pack_reduce(obj);
  }

  void pack_global(PyObject* obj) {
    Ref name = checked(PyObject_GetAttr(obj, s_qualname));
    pack_global_named(obj, std::move(name));
  }

  // `obj` is to be found again as module.name (dotted). Like pickle, check now that the lookup gives this very
  // object: a lambda, a class made inside a function or an object shadowed by another of the same name would
  // otherwise serialize fine and fail (or come back as something else) on the receiving side.
  void pack_global_named(PyObject* obj, Ref name) {
    Ref module;
    if (PyObject* m = PyObject_GetAttr(obj, s_module)) {
      module = Ref(m);
    } else {
      PyErr_Clear();
    }
    if (!module || module.p == Py_None) {
      // singletons such as Ellipsis carry no __module__: ask pickle where the name lives
      Ref pickle_mod = checked(PyImport_ImportModule("pickle"));
      module = checked(PyObject_CallMethod(pickle_mod.p, "whichmodule", "OO", obj, name.p));
    }
    if (!PyUnicode_Check(name.p) || !PyUnicode_Check(module.p)) {
      PyErr_Format(PyExc_TypeError, "moodist.serialize: %R has a name or module that is not a str", obj);
      throw PyError{};
    }
    bool same = false;
    if (PyObject* mod = PyImport_Import(module.p)) {
      Ref cur(mod);
      Ref parts = checked(PyUnicode_Split(name.p, s_dot, -1));
      for (Py_ssize_t i = 0; cur && i < PyList_GET_SIZE(parts.p); ++i)
        cur = Ref(PyObject_GetAttr(cur.p, PyList_GET_ITEM(parts.p, i)));
      same = cur && cur.p == obj;
    }
    if (!same) {
      PyErr_Clear();
      PyErr_Format(PyExc_ValueError, "moodist.serialize: cannot serialize %R: it is not what %U.%U names", obj, module.p,
                   name.p);
      throw PyError{};
    }
    byte(T_GLOBAL);
    pack_temp(std::move(name));
    pack_temp(std::move(module));
  }

  // pack an object we own only temporarily: keep it alive so its address cannot be recycled for
  // another object while it sits in the identity memo
  void pack_temp(Ref r) {
    PyObject* p = r.p;
    keepalive_.push_back(std::move(r));
    pack(p);
  }

  void pack_reduce(PyObject* obj) {
    Ref red;
    // a reducer registered with copyreg.pickle() comes first, as in pickle (re.Pattern is served that way)
    PyObject* registered = g_dispatch_table ? PyDict_GetItemWithError(g_dispatch_table, (PyObject*)Py_TYPE(obj)) : nullptr;
    if (registered) {
      red = checked(PyObject_CallOneArg(registered, obj));
    } else {
      if (PyErr_Occurred()) throw PyError{};
      Ref fn = checked(PyObject_GetAttr(obj, s_reduce_ex));
      red = checked(PyObject_CallOneArg(fn.p, s_five));
    }
    if (PyUnicode_Check(red.p)) return pack_global_named(obj, std::move(red));  // "a global of that name"
    if (!PyTuple_Check(red.p)) {
      PyErr_Format(PyExc_TypeError, "moodist.serialize: %s.__reduce__ must return a tuple or str", Py_TYPE(obj)->tp_name);
      throw PyError{};
    }
    Py_ssize_t n = PyTuple_GET_SIZE(red.p);
    if (n < 2) {
      PyErr_Format(PyExc_TypeError, "moodist.serialize: %s.__reduce__ must return at least (callable, args)",
                   Py_TYPE(obj)->tp_name);
      throw PyError{};
    }
    auto item = [&](Py_ssize_t i) { return i < n ? PyTuple_GET_ITEM(red.p, i) : Py_None; };
    PyObject *func = item(0), *args = item(1), *state = item(2), *listit = item(3), *dictit = item(4), *setstate = item(5);
    PyObject* red_raw = red.p;
    keepalive_.push_back(std::move(red));
    (void)red_raw;
    byte(T_CLASS);
    pack(func);
    pack(args);
    uint8_t bits = (state != Py_None ? 1 : 0) | (listit != Py_None ? 2 : 0) | (dictit != Py_None ? 4 : 0) |
                   (setstate != Py_None ? 8 : 0);
    byte(bits);
    if (bits & 1) {
      pack(state);
      if (bits & 8) pack(setstate);
    }
    if (bits & 2) {
      std::vector<Ref> items;
      while (PyObject* o = PyIter_Next(listit)) items.emplace_back(o);
      if (PyErr_Occurred()) throw PyError{};
      byte(T_LIST);
      pack_int((int64_t)items.size());
      for (Ref& r : items) pack_temp(std::move(r));
    }
    if (bits & 4) {
      size_t at = out.size();
      u64(0);
      uint64_t count = 0;
      while (PyObject* o = PyIter_Next(dictit)) {
        Ref pair(o);
        if (!PyTuple_Check(o) || PyTuple_GET_SIZE(o) != 2) {
          PyErr_SetString(PyExc_TypeError, "moodist.serialize: dict item iterator must yield (key, value) pairs");
          throw PyError{};
        }
        PyObject* k = PyTuple_GET_ITEM(o, 0);
        PyObject* v = PyTuple_GET_ITEM(o, 1);
        keepalive_.push_back(std::move(pair));
        pack(k);
        pack(v);
        ++count;
      }
      if (PyErr_Occurred()) throw PyError{};
      memcpy(out.data() + at, &count, 8);
    }
  }
};

// ------------------------------------------------------------------------------------------------
class Unpacker {
 public:
  Unpacker(const uint8_t* data, size_t n) : base_(data), p_(data), end_(data + n) {}

  size_t consumed() const { return (size_t)(p_ - base_); }

  // returns a new reference
  PyObject* unpack() {
    size_t offset = consumed();
    uint8_t tag = u8();
    bool store = tag & 0x80;
    tag &= 0x7f;
    switch (tag) {
      case T_NONE: Py_RETURN_NONE;
      case T_TRUE: Py_RETURN_TRUE;
      case T_FALSE: Py_RETURN_FALSE;
      case T_INT8: return checked(PyLong_FromLong(read<int8_t>())).release();
      case T_INT16: return checked(PyLong_FromLong(read<int16_t>())).release();
      case T_INT32: return checked(PyLong_FromLong(read<int32_t>())).release();
      case T_INT64: return checked(PyLong_FromLongLong(read<int64_t>())).release();
      case T_FLOAT: return checked(PyFloat_FromDouble(read<double>())).release();
      case T_BIGINT: {
        uint64_t n = read<uint64_t>();
        const uint8_t* b = take(n);
        return checked(_PyLong_FromByteArray(b, n, 1, 1)).release();
      }
      case T_UNICODE: {
        uint8_t kind = u8();
        uint64_t nbytes = read<uint64_t>();
        if (kind != 1 && kind != 2 && kind != 4) bad("bad unicode kind");
        const uint8_t* b = take(nbytes);
        return keep(store, offset, checked(PyUnicode_FromKindAndData(kind, b, (Py_ssize_t)(nbytes / kind))));
      }
      case T_STR:
      case T_BYTES: {
        uint64_t n = read<uint64_t>();
        const uint8_t* b = take(n);
        if (tag == T_STR) return keep(store, offset, checked(PyUnicode_DecodeUTF8((const char*)b, n, nullptr)));
        return keep(store, offset, checked(PyBytes_FromStringAndSize((const char*)b, n)));
      }
      case T_BYTEARRAY: {
        uint64_t n = read<uint64_t>();
        const uint8_t* b = take(n);
        return keep(store, offset, checked(PyByteArray_FromStringAndSize((const char*)b, n)));
      }
      case T_LIST: {
        int64_t n = unpack_len();
        Ref list = checked(PyList_New(n));
        if (store) {
          // The list can be reached through a back reference while it is being filled (it may contain itself).
          // A damaged stream could hand it, half filled, to any callable: no slot is ever left empty.
          for (int64_t i = 0; i < n; ++i) {
            Py_INCREF(Py_None);
            PyList_SET_ITEM(list.p, i, Py_None);
          }
          remember(offset, list.p);
          for (int64_t i = 0; i < n; ++i) {
            PyObject* item = unpack();
            PyObject* placeholder = PyList_GET_ITEM(list.p, i);
            PyList_SET_ITEM(list.p, i, item);
            Py_DECREF(placeholder);
          }
          return list.release();
        }
        for (int64_t i = 0; i < n; ++i) PyList_SET_ITEM(list.p, i, unpack());
        return list.release();
      }
      case T_TUPLE: {
        int64_t n = unpack_len();
        Ref tup = checked(PyTuple_New(n));
        if (store) {
          // A tuple can contain itself through a list, a dict or an object, and the writer then refers to it from
          // inside (as the reference's reader expects, which also stores a tuple before filling it: wrapper/
          // serialize/serialize_object.cc:1034). So a referenced tuple is handed out early like a list, with None
          // in every slot that has no member yet. The collector stops tracking a tuple of atoms if it runs in
          // between; the tuple is tracked again once it is whole, since it may hold containers by then.
          for (int64_t i = 0; i < n; ++i) {
            Py_INCREF(Py_None);
            PyTuple_SET_ITEM(tup.p, i, Py_None);
          }
          remember(offset, tup.p);
          for (int64_t i = 0; i < n; ++i) {
            PyObject* item = unpack();
            PyObject* placeholder = PyTuple_GET_ITEM(tup.p, i);
            PyTuple_SET_ITEM(tup.p, i, item);
            Py_DECREF(placeholder);
          }
          if (!PyObject_GC_IsTracked(tup.p)) PyObject_GC_Track(tup.p);
          return tup.release();
        }
        for (int64_t i = 0; i < n; ++i) PyTuple_SET_ITEM(tup.p, i, unpack());
        return tup.release();
      }
      case T_DICT: {
        int64_t n = unpack_len();
        Ref d = checked(PyDict_New());
        if (store) remember(offset, d.p);
        for (int64_t i = 0; i < n; ++i) {
          Ref k(unpack());
          Ref v(unpack());
          if (PyDict_SetItem(d.p, k.p, v.p) < 0) throw PyError{};
        }
        return d.release();
      }
      case T_SET:
      case T_FROZENSET: {
        uint64_t n = read<uint64_t>();
        if (n > remaining()) bad("set length exceeds buffer");
        Ref s = checked(PySet_New(nullptr));
        if (store && tag == T_SET) remember(offset, s.p);
        for (uint64_t i = 0; i < n; ++i) {
          Ref item(unpack());
          if (PySet_Add(s.p, item.p) < 0) throw PyError{};
        }
        if (tag == T_SET) return s.release();
        Ref fs = checked(PyFrozenSet_New(s.p));
        if (store) remember(offset, fs.p);
        return fs.release();
      }
      case T_GLOBAL: return keep(store, offset, unpack_global());
      case T_CLASS: return unpack_class(store, offset);
      case T_OFFSET: {
        uint64_t off = read<uint64_t>();
        PyObject* found = stored_.find(off);
        if (!found) bad("reference to an object that was not stored");
        Py_INCREF(found);
        return found;
      }
      default: bad("unknown type tag");
    }
    return nullptr;
  }

 private:
  const uint8_t *base_, *p_, *end_;
  OffsetMap stored_;

  [[noreturn]] void bad(const char* what) {
    PyErr_Format(PyExc_ValueError, "moodist.deserialize: %s (at byte %zu)", what, consumed());
    throw PyError{};
  }
  size_t remaining() const { return (size_t)(end_ - p_); }
  const uint8_t* take(uint64_t n) {
    if (n > remaining()) bad("truncated buffer");
    const uint8_t* r = p_;
    p_ += n;
    return r;
  }
  uint8_t u8() { return *take(1); }
  template <typename T>
  T read() {
    T v;
    memcpy(&v, take(sizeof(T)), sizeof(T));
    return v;
  }
  void remember(size_t offset, PyObject* o) { stored_.put(offset, o); }
  PyObject* keep(bool store, size_t offset, Ref r) {
    if (store) remember(offset, r.p);
    return r.release();
  }

  int64_t unpack_len() {
    uint8_t tag = u8() & 0x7f;
    int64_t n;
    switch (tag) {
      case T_NONE: n = 0; break;
      case T_INT8: n = read<int8_t>(); break;
      case T_INT16: n = read<int16_t>(); break;
      case T_INT32: n = read<int32_t>(); break;
      case T_INT64: n = read<int64_t>(); break;
      default: bad("expected a length");
    }
    if (n < 0 || (uint64_t)n > remaining()) bad("length exceeds buffer");
    return n;
  }

  Ref unpack_global() {
    Ref name(unpack());
    Ref module(unpack());
    if (!PyUnicode_Check(name.p) || !PyUnicode_Check(module.p)) bad("global name/module must be str");
    Ref obj = checked(PyImport_Import(module.p));
    Ref parts = checked(PyUnicode_Split(name.p, s_dot, -1));
    for (Py_ssize_t i = 0; i < PyList_GET_SIZE(parts.p); ++i) obj = checked(PyObject_GetAttr(obj.p, PyList_GET_ITEM(parts.p, i)));
    return obj;
  }

  PyObject* unpack_class(bool store, size_t offset) {
    Ref func(unpack());
    Ref args(unpack());
    if (!PyTuple_Check(args.p)) bad("class args must be a tuple");
    Ref obj;
    PyObject* cls = PyTuple_GET_SIZE(args.p) ? PyTuple_GET_ITEM(args.p, 0) : nullptr;
    if (func.p == g_newobj && cls && PyType_Check(cls) && ((PyTypeObject*)cls)->tp_new) {
      // copyreg.__newobj__(cls, *rest) is cls.__new__(cls, *rest): make that call without the Python frame
      Ref rest = checked(PyTuple_GetSlice(args.p, 1, PyTuple_GET_SIZE(args.p)));
      obj = checked(((PyTypeObject*)cls)->tp_new((PyTypeObject*)cls, rest.p, nullptr));
    } else {
      obj = checked(PyObject_Call(func.p, args.p, nullptr));
    }
    if (store) remember(offset, obj.p);
    uint8_t bits = u8();
    if (bits & 1) {
      Ref state(unpack());
      if (bits & 8) {
        Ref setstate(unpack());
        checked(PyObject_CallFunctionObjArgs(setstate.p, obj.p, state.p, nullptr));
      } else if (PyObject_HasAttr(obj.p, s_setstate) && has_custom_setstate(obj.p)) {
        checked(PyObject_CallMethodOneArg(obj.p, s_setstate, state.p));
      } else {
        apply_default_state(obj.p, state.p);
      }
    }
    if (bits & 2) {
      Ref items(unpack());
      if (!PyList_Check(items.p)) bad("list items of an object are not a list");
      if (PyObject_HasAttr(obj.p, s_extend)) {
        checked(PyObject_CallMethodOneArg(obj.p, s_extend, items.p));
      } else {
        for (Py_ssize_t i = 0; i < PyList_GET_SIZE(items.p); ++i)
          checked(PyObject_CallMethodOneArg(obj.p, s_append, PyList_GET_ITEM(items.p, i)));
      }
    }
    if (bits & 4) {
      uint64_t n = read<uint64_t>();
      for (uint64_t i = 0; i < n; ++i) {
        Ref k(unpack());
        Ref v(unpack());
        if (PyObject_SetItem(obj.p, k.p, v.p) < 0) throw PyError{};
      }
    }
    return obj.release();
  }

  static bool has_custom_setstate(PyObject* obj) {
    // object.__setstate__ does not exist before 3.11; from 3.11 on a default one is absent too, so any
    // __setstate__ found is the class's own
    (void)obj;
    return true;
  }

  // pickle's default: state is a dict for __dict__, or (dict_state, slots_state)
  void apply_default_state(PyObject* obj, PyObject* state) {
    PyObject* dstate = state;
    PyObject* slots = nullptr;
    if (PyTuple_Check(state) && PyTuple_GET_SIZE(state) == 2) {
      dstate = PyTuple_GET_ITEM(state, 0);
      slots = PyTuple_GET_ITEM(state, 1);
    }
    if (dstate != Py_None) {
      if (!PyDict_Check(dstate)) bad("object state is not a dict");
      Ref d = checked(PyObject_GetAttr(obj, s_dict));
      Py_ssize_t pos = 0;
      PyObject *k, *v;
      while (PyDict_Next(dstate, &pos, &k, &v)) {
        if (PyUnicode_CheckExact(k)) {
          Py_INCREF(k);
          PyUnicode_InternInPlace(&k);
          int rc = PyObject_SetItem(d.p, k, v);
          Py_DECREF(k);
          if (rc < 0) throw PyError{};
        } else if (PyObject_SetItem(d.p, k, v) < 0) {
          throw PyError{};
        }
      }
    }
    if (slots && slots != Py_None) {
      if (!PyDict_Check(slots)) bad("slots state is not a dict");
      Py_ssize_t pos = 0;
      PyObject *k, *v;
      while (PyDict_Next(slots, &pos, &k, &v))
        if (PyObject_SetAttr(obj, k, v) < 0) throw PyError{};
    }
  }
};

// ------------------------------------------------------------------------------------------------
PyObject* py_pack(PyObject*, PyObject* obj) {
  init_strings();
  try {
    Packer pk;
    pk.out.reserve(256);
    pk.pack(obj);
    return pk.out.release();
  } catch (const PyError&) {
    return nullptr;
  } catch (const std::exception& e) {
    PyErr_SetString(PyExc_RuntimeError, e.what());
    return nullptr;
  }
}

PyObject* py_unpack(PyObject*, PyObject* arg) {
  init_strings();
  Py_buffer view;
  if (PyObject_GetBuffer(arg, &view, PyBUF_SIMPLE) < 0) return nullptr;
  PyObject* result = nullptr;
  try {
    Unpacker up((const uint8_t*)view.buf, (size_t)view.len);
    result = up.unpack();
    if (result && up.consumed() != (size_t)view.len) {
      Py_DECREF(result);
      result = nullptr;
      PyErr_Format(PyExc_ValueError, "moodist.deserialize: %zu trailing bytes", (size_t)view.len - up.consumed());
    }
  } catch (const PyError&) {
    result = nullptr;
  } catch (const std::exception& e) {
    PyErr_SetString(PyExc_RuntimeError, e.what());
    result = nullptr;
  }
  PyBuffer_Release(&view);
  return result;
}

PyMethodDef methods[] = {
    {"pack", py_pack, METH_O, "pack(obj) -> bytearray in the moodist object format"},
    {"unpack", py_unpack, METH_O, "unpack(buffer) -> object"},
    {nullptr, nullptr, 0, nullptr},
};

PyModuleDef module_def = {PyModuleDef_HEAD_INIT, "_serialize", "moodist Python-object serializer", -1, methods,
                          nullptr, nullptr, nullptr, nullptr};

}  // namespace

PyMODINIT_FUNC PyInit__serialize(void) { return PyModule_Create(&module_def); }
