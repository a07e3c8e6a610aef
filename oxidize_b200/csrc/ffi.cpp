// C ABI over the engine: thin entry points that call oxidize_b200.ffi_backend inside an embedded (or the hosting)
// Python interpreter.  Handles are owned references to Python objects.
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>

#include "oxidize_ffi.h"

#ifndef OXIDIZE_DEFAULT_PYTHON
#define OXIDIZE_DEFAULT_PYTHON "python3"
#endif
#ifndef OXIDIZE_DEFAULT_ROOT
#define OXIDIZE_DEFAULT_ROOT ""
#endif

namespace {

std::once_flag g_once;
PyObject* g_backend = nullptr;  // the imported module; never released

void start_interpreter() {
  if (!Py_IsInitialized()) {
    PyConfig config;
    PyConfig_InitPythonConfig(&config);
    const char* exe = std::getenv("OXIDIZE_PYTHON");
    // the interpreter's own path decides which site-packages (a virtual environment's) are found
    PyStatus st = PyConfig_SetBytesString(&config, &config.executable, exe && *exe ? exe : OXIDIZE_DEFAULT_PYTHON);
    if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
    PyConfig_Clear(&config);
    if (PyStatus_Exception(st)) {
      std::fprintf(stderr, "oxidize_ffi: cannot start Python: %s\n", st.err_msg ? st.err_msg : "?");
      return;
    }
    PyEval_SaveThread();  // drop the lock the initialising thread holds; every entry point takes it for its own call
  }
  PyGILState_STATE gil = PyGILState_Ensure();
  const char* root = std::getenv("OXIDIZE_PACKAGE_ROOT");
  std::string r = root && *root ? root : OXIDIZE_DEFAULT_ROOT;
  if (!r.empty()) {
    PyObject* path = PySys_GetObject("path");  // borrowed
    PyObject* s = PyUnicode_FromString(r.c_str());
    if (path && s && !PySequence_Contains(path, s)) PyList_Insert(path, 0, s);
    Py_XDECREF(s);
  }
  g_backend = PyImport_ImportModule("oxidize_b200.ffi_backend");
  if (!g_backend) PyErr_Print();
  PyGILState_Release(gil);
}

struct Gil {
  PyGILState_STATE s;
  bool ok;
  Gil() : ok(false) {
    std::call_once(g_once, start_interpreter);
    if (!g_backend) return;
    s = PyGILState_Ensure();
    ok = true;
  }
  ~Gil() {
    if (ok) PyGILState_Release(s);
  }
};

// call backend.<name>(args...) -> new reference or nullptr (error printed)
PyObject* call(const char* name, const char* fmt, ...) {
  PyObject* fn = PyObject_GetAttrString(g_backend, name);
  if (!fn) {
    PyErr_Print();
    return nullptr;
  }
  va_list va;
  va_start(va, fmt);
  PyObject* args = Py_VaBuildValue(fmt, va);
  va_end(va);
  PyObject* out = nullptr;
  if (args) {
    if (!PyTuple_Check(args)) {  // a single argument comes back bare
      PyObject* t = PyTuple_Pack(1, args);
      Py_DECREF(args);
      args = t;
    }
    if (args) out = PyObject_CallObject(fn, args);
  }
  if (!out) PyErr_Print();
  Py_XDECREF(args);
  Py_DECREF(fn);
  return out;
}

long as_long(PyObject* o, long on_error) {
  if (!o) return on_error;
  long v = PyLong_AsLong(o);
  if (v == -1 && PyErr_Occurred()) {
    PyErr_Print();
    v = on_error;
  }
  Py_DECREF(o);
  return v;
}

}  // namespace

extern "C" {

const char* oxidize_ffi_version(void) { return "oxidize-b200-ffi 1"; }

int32_t oxidize_gemv_quantized(uint32_t quant_type, const uint8_t* qbytes, size_t qbytes_len, size_t rows, size_t cols,
                               const float* vector, float* output) {
  if (!qbytes || !vector || !output) return -2;
  Gil g;
  if (!g.ok) return -1;
  return (int32_t)as_long(call("gemv_quantized", "(IKKKKKK)", quant_type, (unsigned long long)(uintptr_t)qbytes,
                               (unsigned long long)qbytes_len, (unsigned long long)rows, (unsigned long long)cols,
                               (unsigned long long)(uintptr_t)vector, (unsigned long long)(uintptr_t)output), -1);
}

void* oxidize_model_load(const char* path) {
  if (!path) return nullptr;
  Gil g;
  if (!g.ok) return nullptr;
  return call("model_load", "(s)", path);  // the new reference is the handle
}

void oxidize_model_free(void* model) {
  if (!model) return;
  Gil g;
  if (g.ok) Py_DECREF(reinterpret_cast<PyObject*>(model));
}

uint32_t oxidize_model_vocab_size(void* model) {
  if (!model) return 0;
  Gil g;
  if (!g.ok) return 0;
  return (uint32_t)as_long(call("model_vocab_size", "(O)", reinterpret_cast<PyObject*>(model)), 0);
}

void* oxidize_session_new(void) {
  Gil g;
  if (!g.ok) return nullptr;
  return call("session_new", "()");
}

void oxidize_session_reset(void* session) {
  if (!session) return;
  Gil g;
  if (!g.ok) return;
  PyObject* r = PyObject_CallMethod(reinterpret_cast<PyObject*>(session), "reset", nullptr);
  if (!r) PyErr_Print();
  Py_XDECREF(r);
}

void oxidize_session_free(void* session) {
  if (!session) return;
  oxidize_session_reset(session);
  Gil g;
  if (g.ok) Py_DECREF(reinterpret_cast<PyObject*>(session));
}

int32_t oxidize_model_forward(void* model, void* session, const uint32_t* tokens, size_t n_tokens, float* logits_out,
                              size_t vocab_size) {
  if (!model || !session || !tokens || !logits_out || n_tokens == 0) return -2;
  Gil g;
  if (!g.ok) return -1;
  PyObject* list = PyList_New((Py_ssize_t)n_tokens);
  if (!list) return -1;
  for (size_t i = 0; i < n_tokens; ++i) PyList_SET_ITEM(list, (Py_ssize_t)i, PyLong_FromUnsignedLong(tokens[i]));
  PyObject* out = call("model_forward", "(OOOKK)", reinterpret_cast<PyObject*>(model), reinterpret_cast<PyObject*>(session),
                       list, (unsigned long long)(uintptr_t)logits_out, (unsigned long long)vocab_size);
  Py_DECREF(list);
  return (int32_t)as_long(out, -1);
}

uint32_t oxidize_sample_argmax(const float* logits, size_t vocab_size) {
  if (!logits || vocab_size == 0) return 0;
  size_t best = 0;
  for (size_t i = 1; i < vocab_size; ++i)
    if (logits[i] >= logits[best]) best = i;  // the last maximal element
  return (uint32_t)best;
}

}  // extern "C"
