// Implementation of xllm.h on top of an embedded (or already running) CPython interpreter.
#include "xllm.h"

#include <Python.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

struct xllm_llm {
  PyObject* handle;  // object returned by c_bridge.create
};

namespace {
std::string g_error;
std::once_flag g_init;
bool g_we_initialised = false;

void ensure_python() {
  std::call_once(g_init, [] {
    if (!Py_IsInitialized()) {
      Py_InitializeEx(0);
      g_we_initialised = true;
      PyEval_SaveThread();  // release the GIL: every entry point takes it with PyGILState_Ensure
    }
  });
}

struct Gil {
  PyGILState_STATE st;
  Gil() : st(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(st); }
};

void take_error(const char* what) {
  g_error = what;
  if (PyErr_Occurred()) {
    PyObject *t, *v, *tb;
    PyErr_Fetch(&t, &v, &tb);
    PyErr_NormalizeException(&t, &v, &tb);
    if (v != nullptr) {
      PyObject* s = PyObject_Str(v);
      if (s != nullptr) {
        const char* c = PyUnicode_AsUTF8(s);
        if (c != nullptr) g_error += std::string(": ") + c;
        Py_DECREF(s);
      }
    }
    Py_XDECREF(t);
    Py_XDECREF(v);
    Py_XDECREF(tb);
  }
}

PyObject* bridge(const char* fn) {
  PyObject* mod = PyImport_ImportModule("xllm_b200.api.c_bridge");
  if (mod == nullptr) return nullptr;
  PyObject* f = PyObject_GetAttrString(mod, fn);
  Py_DECREF(mod);
  return f;
}

char* dup_result(PyObject* r) {
  if (r == nullptr) return nullptr;
  const char* c = PyUnicode_AsUTF8(r);
  char* out = c != nullptr ? strdup(c) : nullptr;
  Py_DECREF(r);
  return out;
}
}  // namespace

extern "C" {

xllm_llm* xllm_llm_create(const char* model, const char* options_json) {
  ensure_python();
  Gil gil;
  PyObject* f = bridge("create");
  if (f == nullptr) {
    take_error("cannot import xllm_b200.api.c_bridge");
    return nullptr;
  }
  PyObject* h = PyObject_CallFunction(f, "ss", model ? model : "tiny", options_json ? options_json : "{}");
  Py_DECREF(f);
  if (h == nullptr) {
    take_error("xllm_llm_create failed");
    return nullptr;
  }
  xllm_llm* llm = new xllm_llm{h};
  return llm;
}

void xllm_llm_destroy(xllm_llm* llm) {
  if (llm == nullptr) return;
  {
    Gil gil;
    Py_XDECREF(llm->handle);
  }
  delete llm;
}

char* xllm_llm_generate(xllm_llm* llm, const char* prompts_json, const char* sampling_json) {
  if (llm == nullptr || prompts_json == nullptr) {
    g_error = "null argument";
    return nullptr;
  }
  Gil gil;
  PyObject* f = bridge("generate");
  if (f == nullptr) {
    take_error("cannot import xllm_b200.api.c_bridge");
    return nullptr;
  }
  PyObject* r = PyObject_CallFunction(f, "Oss", llm->handle, prompts_json, sampling_json ? sampling_json : "{}");
  Py_DECREF(f);
  if (r == nullptr) {
    take_error("xllm_llm_generate failed");
    return nullptr;
  }
  return dup_result(r);
}

char* xllm_llm_stats(xllm_llm* llm) {
  if (llm == nullptr) return nullptr;
  Gil gil;
  PyObject* f = bridge("stats");
  if (f == nullptr) {
    take_error("cannot import xllm_b200.api.c_bridge");
    return nullptr;
  }
  PyObject* r = PyObject_CallFunction(f, "O", llm->handle);
  Py_DECREF(f);
  if (r == nullptr) {
    take_error("xllm_llm_stats failed");
    return nullptr;
  }
  return dup_result(r);
}

char* xllm_llm_call(xllm_llm* llm, const char* method, const char* args_json) {
  if (llm == nullptr || method == nullptr) {
    g_error = "null argument";
    return nullptr;
  }
  Gil gil;
  PyObject* f = bridge("call");
  if (f == nullptr) {
    take_error("cannot import xllm_b200.api.c_bridge");
    return nullptr;
  }
  PyObject* r = PyObject_CallFunction(f, "Oss", llm->handle, method, args_json ? args_json : "{}");
  Py_DECREF(f);
  if (r == nullptr) {
    take_error("xllm_llm_call failed");
    return nullptr;
  }
  return dup_result(r);
}

void xllm_free_string(char* s) { free(s); }
const char* xllm_last_error(void) { return g_error.c_str(); }

}  // extern "C"
