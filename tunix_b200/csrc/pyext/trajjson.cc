// _trajjson: GIL-free serialisation of trajectory objects (CPython extension module).
//
//   format_ndarray(arr) -> str     text identical to repr(arr.tolist()): "[1, 2.5, True]", nested brackets
//   dumps_json(obj, indent=-1) -> str   json.dumps-compatible output for dict / list / tuple / str / int /
//                                       float / bool / None / dataclasses / numpy scalars and arrays,
//                                       ensure_ascii escaping, NaN / Infinity tokens, optional indent
//   SerializedArray(str)           str subclass whose repr() is the unquoted text; dumps_json emits it raw
//
// Two phases: with the GIL held the Python tree is converted to a plain C++ node tree (array payloads are
// referenced through the buffer protocol, not copied); the text is produced with the GIL released.
// Doubles print as Python's float.__repr__: shortest round-trip digits, fixed notation for
// -4 <= exp10 < 16, otherwise scientific with a sign and at least two exponent digits.
// float32 arrays are widened to double first (what arr.tolist() shows).
//
// Same role as the reference's trajectory-logger extension (tunix/utils/_trajectory_logger_ext.cc:149-212
// float repr, :238-405 ndarray formatter, :532-791 JSON tree + emit).
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <charconv>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace {

void append_double(std::string& out, double v, bool json) {
  if (std::isnan(v)) { out += json ? "NaN" : "nan"; return; }
  if (std::isinf(v)) { out += v > 0 ? (json ? "Infinity" : "inf") : (json ? "-Infinity" : "-inf"); return; }
  if (v == 0.0) { out += std::signbit(v) ? "-0.0" : "0.0"; return; }
  char buf[64];
  auto res = std::to_chars(buf, buf + sizeof(buf), v, std::chars_format::scientific);
  std::string s(buf, res.ptr);          // d.ddddde[+-]XX, shortest round-trip
  size_t epos = s.find('e');
  std::string mant = s.substr(0, epos);
  int exp10 = std::stoi(s.substr(epos + 1));
  bool neg = false;
  if (mant[0] == '-') { neg = true; mant = mant.substr(1); }
  std::string digits;
  for (char c : mant) if (c != '.') digits.push_back(c);
  if (neg) out.push_back('-');
  if (exp10 >= -4 && exp10 < 16) {
    if (exp10 >= 0) {
      size_t int_len = (size_t)exp10 + 1;
      if (digits.size() <= int_len) {
        out += digits;
        out.append(int_len - digits.size(), '0');
        out += ".0";
      } else {
        out.append(digits, 0, int_len);
        out.push_back('.');
        out.append(digits, int_len, std::string::npos);
      }
    } else {
      out += "0.";
      out.append((size_t)(-exp10 - 1), '0');
      out += digits;
    }
  } else {
    out.push_back(digits[0]);
    if (digits.size() > 1) { out.push_back('.'); out.append(digits, 1, std::string::npos); }
    out.push_back('e');
    out.push_back(exp10 < 0 ? '-' : '+');
    int a = exp10 < 0 ? -exp10 : exp10;
    if (a < 10) out.push_back('0');
    out += std::to_string(a);
  }
}

enum class DT { I8, I16, I32, I64, U8, U16, U32, U64, F32, F64, BOOL, UNKNOWN };

DT parse_format(const char* f, Py_ssize_t itemsize) {
  if (!f) return DT::UNKNOWN;
  while (*f == '<' || *f == '=' || *f == '@' || *f == '|') ++f;
  if (*f == '>' || *f == '!') return DT::UNKNOWN;
  switch (*f) {
    case 'b': return DT::I8;
    case 'B': return DT::U8;
    case 'h': return DT::I16;
    case 'H': return DT::U16;
    case 'i': return DT::I32;
    case 'I': return DT::U32;
    case 'l': return itemsize == 8 ? DT::I64 : DT::I32;
    case 'L': return itemsize == 8 ? DT::U64 : DT::U32;
    case 'q': return DT::I64;
    case 'Q': return DT::U64;
    case 'f': return DT::F32;
    case 'd': return DT::F64;
    case '?': return DT::BOOL;
    default: return DT::UNKNOWN;
  }
}

struct ArrayView {
  Py_buffer buf;
  bool held = false;
  DT dt = DT::UNKNOWN;
  ~ArrayView() {}
};

void emit_element(std::string& out, const char* p, DT dt, bool json) {
  switch (dt) {
    case DT::I8: out += std::to_string((int)*(const int8_t*)p); break;
    case DT::I16: { int16_t v; memcpy(&v, p, 2); out += std::to_string(v); break; }
    case DT::I32: { int32_t v; memcpy(&v, p, 4); out += std::to_string(v); break; }
    case DT::I64: { int64_t v; memcpy(&v, p, 8); out += std::to_string(v); break; }
    case DT::U8: out += std::to_string((unsigned)*(const uint8_t*)p); break;
    case DT::U16: { uint16_t v; memcpy(&v, p, 2); out += std::to_string(v); break; }
    case DT::U32: { uint32_t v; memcpy(&v, p, 4); out += std::to_string(v); break; }
    case DT::U64: { uint64_t v; memcpy(&v, p, 8); out += std::to_string(v); break; }
    case DT::F32: { float v; memcpy(&v, p, 4); append_double(out, (double)v, json); break; }
    case DT::F64: { double v; memcpy(&v, p, 8); append_double(out, v, json); break; }
    case DT::BOOL: out += (*p ? (json ? "true" : "True") : (json ? "false" : "False")); break;
    default: out += "null";
  }
}

void emit_array(std::string& out, const Py_buffer& b, DT dt, int dim, const char* base, bool json) {
  if (b.ndim == 0) { emit_element(out, base, dt, json); return; }
  const Py_ssize_t n = b.shape[dim];
  const Py_ssize_t stride = b.strides ? b.strides[dim] : 0;
  out.push_back('[');
  for (Py_ssize_t i = 0; i < n; ++i) {
    if (i) out += ", ";
    const char* p = base + i * stride;
    if (dim + 1 == b.ndim) emit_element(out, p, dt, json);
    else emit_array(out, b, dt, dim + 1, p, json);
  }
  out.push_back(']');
}

// ----------------------------------------------------------------- JSON node tree
struct Node {
  enum Kind { NUL, TRUE_, FALSE_, INT, DBL, STR, RAW, LIST, DICT, ARRAY } kind = NUL;
  std::string text;                    // INT digits, STR utf-8, RAW preformatted
  double dbl = 0;
  std::vector<std::unique_ptr<Node>> items;      // LIST values / DICT values
  std::vector<std::string> keys;                 // DICT keys (utf-8)
  std::shared_ptr<ArrayView> arr;
};

void escape_string(std::string& out, const std::string& s) {
  out.push_back('"');
  const unsigned char* p = (const unsigned char*)s.data();
  const unsigned char* end = p + s.size();
  char buf[16];
  while (p < end) {
    uint32_t c = *p;
    int len = 1;
    if (c >= 0xF0 && p + 3 < end + 0) { c = ((c & 7) << 18) | ((p[1] & 0x3F) << 12) | ((p[2] & 0x3F) << 6) | (p[3] & 0x3F); len = 4; }
    else if (c >= 0xE0) { c = ((c & 0xF) << 12) | ((p[1] & 0x3F) << 6) | (p[2] & 0x3F); len = 3; }
    else if (c >= 0xC0) { c = ((c & 0x1F) << 6) | (p[1] & 0x3F); len = 2; }
    p += len;
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      case '\b': out += "\\b"; break;
      case '\f': out += "\\f"; break;
      default:
        if (c < 0x20 || c > 0x7E) {
          if (c >= 0x10000) {
            uint32_t v = c - 0x10000;
            snprintf(buf, sizeof(buf), "\\u%04x\\u%04x", 0xD800 + (v >> 10), 0xDC00 + (v & 0x3FF));
          } else {
            snprintf(buf, sizeof(buf), "\\u%04x", c);
          }
          out += buf;
        } else {
          out.push_back((char)c);
        }
    }
  }
  out.push_back('"');
}

void newline(std::string& out, int indent, int depth) {
  if (indent < 0) return;
  out.push_back('\n');
  out.append((size_t)indent * depth, ' ');
}

void emit_node(std::string& out, const Node& n, int indent, int depth) {
  switch (n.kind) {
    case Node::NUL: out += "null"; break;
    case Node::TRUE_: out += "true"; break;
    case Node::FALSE_: out += "false"; break;
    case Node::INT: out += n.text; break;
    case Node::DBL: append_double(out, n.dbl, true); break;
    case Node::STR: escape_string(out, n.text); break;
    case Node::RAW: out += n.text; break;
    case Node::ARRAY: emit_array(out, n.arr->buf, n.arr->dt, 0, (const char*)n.arr->buf.buf, true); break;
    case Node::LIST:
      if (n.items.empty()) { out += "[]"; break; }
      out.push_back('[');
      for (size_t i = 0; i < n.items.size(); ++i) {
        if (i) out += indent < 0 ? ", " : ",";
        newline(out, indent, depth + 1);
        emit_node(out, *n.items[i], indent, depth + 1);
      }
      newline(out, indent, depth);
      out.push_back(']');
      break;
    case Node::DICT:
      if (n.items.empty()) { out += "{}"; break; }
      out.push_back('{');
      for (size_t i = 0; i < n.items.size(); ++i) {
        if (i) out += indent < 0 ? ", " : ",";
        newline(out, indent, depth + 1);
        escape_string(out, n.keys[i]);
        out += ": ";
        emit_node(out, *n.items[i], indent, depth + 1);
      }
      newline(out, indent, depth);
      out.push_back('}');
      break;
  }
}

PyObject* g_serialized_array_type = nullptr;
PyObject* g_dataclasses = nullptr;

bool utf8_of(PyObject* s, std::string& out) {
  Py_ssize_t n;
  const char* p = PyUnicode_AsUTF8AndSize(s, &n);
  if (!p) return false;
  out.assign(p, (size_t)n);
  return true;
}

std::unique_ptr<Node> build(PyObject* o, std::vector<std::shared_ptr<ArrayView>>& views, int depth);

std::unique_ptr<Node> build_from_str_fallback(PyObject* o) {
  auto n = std::make_unique<Node>();
  PyObject* s = PyObject_Str(o);
  if (!s) return nullptr;
  n->kind = Node::STR;
  bool ok = utf8_of(s, n->text);
  Py_DECREF(s);
  return ok ? std::move(n) : nullptr;
}

std::unique_ptr<Node> build(PyObject* o, std::vector<std::shared_ptr<ArrayView>>& views, int depth) {
  if (depth > 200) { PyErr_SetString(PyExc_RecursionError, "object nested too deeply"); return nullptr; }
  auto n = std::make_unique<Node>();
  if (o == Py_None) { n->kind = Node::NUL; return n; }
  if (o == Py_True) { n->kind = Node::TRUE_; return n; }
  if (o == Py_False) { n->kind = Node::FALSE_; return n; }
  if (g_serialized_array_type && PyObject_IsInstance(o, g_serialized_array_type) == 1) {
    n->kind = Node::RAW;
    if (!utf8_of(o, n->text)) return nullptr;
    return n;
  }
  if (PyLong_Check(o)) {
    PyObject* s = PyObject_Str(o);
    if (!s) return nullptr;
    n->kind = Node::INT;
    bool ok = utf8_of(s, n->text);
    Py_DECREF(s);
    return ok ? std::move(n) : nullptr;
  }
  if (PyFloat_Check(o)) { n->kind = Node::DBL; n->dbl = PyFloat_AS_DOUBLE(o); return n; }
  if (PyUnicode_Check(o)) { n->kind = Node::STR; if (!utf8_of(o, n->text)) return nullptr; return n; }
  if (PyDict_Check(o)) {
    n->kind = Node::DICT;
    PyObject *k, *v;
    Py_ssize_t pos = 0;
    while (PyDict_Next(o, &pos, &k, &v)) {
      std::string key;
      if (PyUnicode_Check(k)) { if (!utf8_of(k, key)) return nullptr; }
      else if (k == Py_True) key = "true";
      else if (k == Py_False) key = "false";
      else if (k == Py_None) key = "null";
      else {
        PyObject* ks = PyObject_Str(k);
        if (!ks) return nullptr;
        bool ok = utf8_of(ks, key);
        Py_DECREF(ks);
        if (!ok) return nullptr;
      }
      auto child = build(v, views, depth + 1);
      if (!child) return nullptr;
      n->keys.push_back(std::move(key));
      n->items.push_back(std::move(child));
    }
    return n;
  }
  if (PyList_Check(o) || PyTuple_Check(o)) {
    n->kind = Node::LIST;
    PyObject* seq = PySequence_Fast(o, "sequence expected");
    if (!seq) return nullptr;
    Py_ssize_t len = PySequence_Fast_GET_SIZE(seq);
    for (Py_ssize_t i = 0; i < len; ++i) {
      auto child = build(PySequence_Fast_GET_ITEM(seq, i), views, depth + 1);
      if (!child) { Py_DECREF(seq); return nullptr; }
      n->items.push_back(std::move(child));
    }
    Py_DECREF(seq);
    return n;
  }
  // dataclass instance -> dict of its fields, in declaration order
  if (g_dataclasses && PyObject_HasAttrString(o, "__dataclass_fields__") && !PyType_Check(o)) {
    PyObject* d = PyObject_CallMethod(g_dataclasses, "asdict", "O", o);
    if (!d) return nullptr;
    auto child = build(d, views, depth + 1);
    Py_DECREF(d);
    return child;
  }
  // numpy scalar -> python scalar via .item(); ndarray via the buffer protocol
  if (PyObject_CheckBuffer(o) && !PyBytes_Check(o) && !PyByteArray_Check(o)) {
    auto view = std::make_shared<ArrayView>();
    if (PyObject_GetBuffer(o, &view->buf, PyBUF_STRIDES | PyBUF_FORMAT) == 0) {
      view->held = true;
      view->dt = parse_format(view->buf.format, view->buf.itemsize);
      if (view->dt != DT::UNKNOWN) {
        views.push_back(view);
        n->kind = Node::ARRAY;
        n->arr = view;
        return n;
      }
      PyBuffer_Release(&view->buf);
      view->held = false;
    } else {
      PyErr_Clear();
    }
    if (PyObject_HasAttrString(o, "tolist")) {
      PyObject* l = PyObject_CallMethod(o, "tolist", nullptr);
      if (!l) return nullptr;
      auto child = build(l, views, depth + 1);
      Py_DECREF(l);
      return child;
    }
  }
  if (PyObject_HasAttrString(o, "item") && PyObject_HasAttrString(o, "dtype")) {
    PyObject* it = PyObject_CallMethod(o, "item", nullptr);
    if (it) {
      auto child = build(it, views, depth + 1);
      Py_DECREF(it);
      return child;
    }
    PyErr_Clear();
  }
  return build_from_str_fallback(o);
}

void release_views(std::vector<std::shared_ptr<ArrayView>>& views) {
  for (auto& v : views)
    if (v->held) { PyBuffer_Release(&v->buf); v->held = false; }
}

PyObject* py_dumps_json(PyObject*, PyObject* args, PyObject* kwargs) {
  PyObject* obj;
  int indent = -1;
  static const char* kw[] = {"obj", "indent", nullptr};
  if (!PyArg_ParseTupleAndKeywords(args, kwargs, "O|i", const_cast<char**>(kw), &obj, &indent)) return nullptr;
  std::vector<std::shared_ptr<ArrayView>> views;
  auto root = build(obj, views, 0);
  if (!root) { release_views(views); return nullptr; }
  std::string out;
  Py_BEGIN_ALLOW_THREADS
  out.reserve(1024);
  emit_node(out, *root, indent, 0);
  root.reset();
  Py_END_ALLOW_THREADS
  release_views(views);
  return PyUnicode_DecodeUTF8(out.data(), (Py_ssize_t)out.size(), "strict");
}

PyObject* py_format_ndarray(PyObject*, PyObject* args) {
  PyObject* obj;
  if (!PyArg_ParseTuple(args, "O", &obj)) return nullptr;
  Py_buffer b;
  if (PyObject_GetBuffer(obj, &b, PyBUF_STRIDES | PyBUF_FORMAT) != 0) return nullptr;
  DT dt = parse_format(b.format, b.itemsize);
  if (dt == DT::UNKNOWN) {
    PyBuffer_Release(&b);
    PyErr_SetString(PyExc_TypeError, "unsupported dtype for format_ndarray");
    return nullptr;
  }
  std::string out;
  Py_BEGIN_ALLOW_THREADS
  emit_array(out, b, dt, 0, (const char*)b.buf, false);
  Py_END_ALLOW_THREADS
  PyBuffer_Release(&b);
  return PyUnicode_DecodeUTF8(out.data(), (Py_ssize_t)out.size(), "strict");
}

PyObject* py_set_serialized_array_type(PyObject*, PyObject* args) {
  PyObject* t;
  if (!PyArg_ParseTuple(args, "O", &t)) return nullptr;
  Py_XDECREF(g_serialized_array_type);
  Py_INCREF(t);
  g_serialized_array_type = t;
  Py_RETURN_NONE;
}

PyMethodDef methods[] = {
    {"dumps_json", (PyCFunction)(void (*)(void))py_dumps_json, METH_VARARGS | METH_KEYWORDS,
     "dumps_json(obj, indent=-1) -> str"},
    {"format_ndarray", py_format_ndarray, METH_VARARGS, "format_ndarray(arr) -> str"},
    {"_set_serialized_array_type", py_set_serialized_array_type, METH_VARARGS, "register the str subclass emitted raw"},
    {nullptr, nullptr, 0, nullptr}};

PyModuleDef moddef = {PyModuleDef_HEAD_INIT, "_trajjson", "GIL-free trajectory serialisation", -1, methods};

}  // namespace

PyMODINIT_FUNC PyInit__trajjson(void) {
  PyObject* m = PyModule_Create(&moddef);
  if (!m) return nullptr;
  g_dataclasses = PyImport_ImportModule("dataclasses");
  if (!g_dataclasses) PyErr_Clear();
  return m;
}
