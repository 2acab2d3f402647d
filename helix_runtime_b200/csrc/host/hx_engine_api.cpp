// The engine for C and C++ callers (include/helix_b200/engine.h): an embedded interpreter
// that hosts the package, one engine object per handle, and plain-value conversions.
//
// Every entry point takes the interpreter's lock, calls one function of
// helix_runtime_b200/capi.py and converts its plain result.  A Python exception becomes the
// error code with the exception's text as the message.
#include <Python.h>

#include "../../../include/helix_b200/engine.h"

#include <dlfcn.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace {

thread_local std::string g_error;
std::once_flag g_started;
std::string g_start_error;
PyObject* g_glue = nullptr;        // the module helix_runtime_b200.capi

int fail(const std::string& message) {
  g_error = message;
  return HXE_ERROR;
}

// The text of the pending Python exception (cleared).
std::string python_error() {
  PyObject *type = nullptr, *value = nullptr, *trace = nullptr;
  PyErr_Fetch(&type, &value, &trace);
  PyErr_NormalizeException(&type, &value, &trace);
  std::string text = "unknown Python error";
  if (value != nullptr) {
    PyObject* shown = PyObject_Str(value);
    if (shown != nullptr) {
      const char* utf8 = PyUnicode_AsUTF8(shown);
      if (utf8 != nullptr) text = utf8;
      Py_DECREF(shown);
    }
    if (type != nullptr) {
      PyObject* name = PyObject_GetAttrString(type, "__name__");
      if (name != nullptr) {
        const char* utf8 = PyUnicode_AsUTF8(name);
        if (utf8 != nullptr) text = std::string(utf8) + ": " + text;
        Py_DECREF(name);
      }
    }
  }
  PyErr_Clear();
  Py_XDECREF(type);
  Py_XDECREF(value);
  Py_XDECREF(trace);
  return text;
}

// The folder that holds the package: this library lives in <root>/helix_runtime_b200/csrc/_build.
std::string package_root() {
  Dl_info info{};
  if (dladdr(reinterpret_cast<const void*>(&package_root), &info) == 0 || info.dli_fname == nullptr)
    return "";
  std::string path = info.dli_fname;
  for (int up = 0; up < 4; ++up) {
    const size_t slash = path.find_last_of('/');
    if (slash == std::string::npos) return "";
    path.erase(slash);
  }
  return path;
}

std::string interpreter_path() {
  if (const char* named = std::getenv("HELIX_B200_PYTHON")) return named;
  const char* search = std::getenv("PATH");
  std::string paths = search != nullptr ? search : "/usr/bin:/bin";
  size_t begin = 0;
  while (begin <= paths.size()) {
    const size_t end = paths.find(':', begin);
    const std::string folder = paths.substr(begin, end == std::string::npos ? end : end - begin);
    const std::string candidate = folder + "/python3";
    if (!folder.empty() && access(candidate.c_str(), X_OK) == 0) return candidate;
    if (end == std::string::npos) break;
    begin = end + 1;
  }
  return "python3";
}

// Start the interpreter (unless the process already runs one) and import the glue module.
void start() {
  const bool ours = !Py_IsInitialized();
  if (ours) {
    PyConfig config;
    PyConfig_InitPythonConfig(&config);
    const std::string program = interpreter_path();
    PyStatus status = PyConfig_SetBytesString(&config, &config.executable, program.c_str());
    if (!PyStatus_Exception(status))
      status = PyConfig_SetBytesString(&config, &config.program_name, program.c_str());
    if (!PyStatus_Exception(status)) status = Py_InitializeFromConfig(&config);
    PyConfig_Clear(&config);
    if (PyStatus_Exception(status)) {
      g_start_error = std::string("could not start Python (") + program + "): " +
                      (status.err_msg != nullptr ? status.err_msg : "unknown error");
      return;
    }
  }
  PyGILState_STATE lock = PyGILState_STATE();
  if (!ours) lock = PyGILState_Ensure();
  const std::string root = package_root();
  PyObject* path = PySys_GetObject("path");      // borrowed
  if (path != nullptr && !root.empty()) {
    PyObject* entry = PyUnicode_FromString(root.c_str());
    if (entry != nullptr) {
      if (PySequence_Contains(path, entry) == 0) PyList_Insert(path, 0, entry);
      Py_DECREF(entry);
    }
  }
  g_glue = PyImport_ImportModule("helix_runtime_b200.capi");
  if (g_glue == nullptr)
    g_start_error = "could not import helix_runtime_b200 from " + root + ": " + python_error();
  if (ours) {
    PyEval_SaveThread();           // leave the lock to the entry points
  } else {
    PyGILState_Release(lock);
  }
}

bool ready() {
  std::call_once(g_started, start);
  if (!g_start_error.empty()) {
    g_error = g_start_error;
    return false;
  }
  return true;
}

struct Locked {
  PyGILState_STATE state;
  Locked() : state(PyGILState_Ensure()) {}
  ~Locked() { PyGILState_Release(state); }
};

// Call glue.<name>(*arguments); steals `arguments`; null on error (message set).
PyObject* call(const char* name, PyObject* arguments) {
  if (arguments == nullptr) {
    g_error = python_error();
    return nullptr;
  }
  PyObject* function = PyObject_GetAttrString(g_glue, name);
  PyObject* result = function != nullptr ? PyObject_CallObject(function, arguments) : nullptr;
  Py_XDECREF(function);
  Py_DECREF(arguments);
  if (result == nullptr) g_error = python_error();
  return result;
}

void copy_text(char* out, size_t capacity, PyObject* text) {
  const char* utf8 = PyUnicode_Check(text) ? PyUnicode_AsUTF8(text) : nullptr;
  std::snprintf(out, capacity, "%s", utf8 != nullptr ? utf8 : "");
  PyErr_Clear();
}

}  // namespace

struct hxe_engine {
  PyObject* object;
};

extern "C" {

const char* hxe_last_error(void) { return g_error.c_str(); }

int hxe_engine_create(const char* model, const hxe_config* config, hxe_engine** out) {
  *out = nullptr;
  if (model == nullptr) return fail("hxe_engine_create: no model path");
  if (!ready()) return HXE_ERROR;
  hxe_config c{};
  if (config != nullptr) c = *config;
  Locked lock;
  PyObject* object = call("create", Py_BuildValue(
      "(ssiiiiiiiii)", model, c.dtype != nullptr ? c.dtype : "bfloat16", c.device,
      c.page_size > 0 ? c.page_size : 16, c.num_pages,
      c.max_running_requests > 0 ? c.max_running_requests : 8,
      c.max_tokens_per_iteration > 0 ? c.max_tokens_per_iteration : 2048, c.max_prefill_chunk,
      c.prefix_cache_entries, c.no_cuda_graphs ? 0 : 1, c.no_lookahead ? 0 : 1));
  if (object == nullptr) return HXE_ERROR;
  *out = new hxe_engine{object};
  return HXE_OK;
}

void hxe_engine_destroy(hxe_engine* engine) {
  if (engine == nullptr) return;
  {
    Locked lock;
    Py_XDECREF(engine->object);
  }
  delete engine;
}

long long hxe_submit(hxe_engine* engine, const int32_t* prompt, int prompt_tokens,
                     int max_new_tokens, int eos_token, float temperature, uint64_t seed) {
  if (engine == nullptr || (prompt == nullptr && prompt_tokens > 0) || prompt_tokens < 0)
    return fail("hxe_submit: bad arguments");
  Locked lock;
  PyObject* tokens = PyList_New(prompt_tokens);
  if (tokens == nullptr) return fail(python_error());
  for (int i = 0; i < prompt_tokens; ++i) PyList_SET_ITEM(tokens, i, PyLong_FromLong(prompt[i]));
  PyObject* id = call("submit", Py_BuildValue("(ONiidK)", engine->object, tokens, max_new_tokens,
                                              eos_token, static_cast<double>(temperature),
                                              static_cast<unsigned long long>(seed)));
  if (id == nullptr) return HXE_ERROR;
  const long long value = PyLong_AsLongLong(id);
  Py_DECREF(id);
  return value;
}

int hxe_run_iteration(hxe_engine* engine, hxe_iteration* out) {
  if (engine == nullptr || out == nullptr) return fail("hxe_run_iteration: bad arguments");
  Locked lock;
  PyObject* result = call("run_iteration", Py_BuildValue("(O)", engine->object));
  if (result == nullptr) return HXE_ERROR;
  const int parsed = PyArg_ParseTuple(result, "iiiiiiii", &out->idle, &out->scheduled_tokens,
                                      &out->prefill_tokens, &out->decode_tokens, &out->sampled,
                                      &out->retired, &out->preempted, &out->kv_limited);
  Py_DECREF(result);
  return parsed ? HXE_OK : fail(python_error());
}

int hxe_run_until_done(hxe_engine* engine, long long max_iterations, long long* iterations) {
  if (engine == nullptr) return fail("hxe_run_until_done: no engine");
  Locked lock;
  PyObject* result = call("run_until_done", Py_BuildValue("(OL)", engine->object, max_iterations));
  if (result == nullptr) return HXE_ERROR;
  if (iterations != nullptr) *iterations = PyLong_AsLongLong(result);
  Py_DECREF(result);
  return HXE_OK;
}

int hxe_cancel(hxe_engine* engine, long long request) {
  if (engine == nullptr) return fail("hxe_cancel: no engine");
  Locked lock;
  PyObject* result = call("cancel", Py_BuildValue("(OL)", engine->object, request));
  if (result == nullptr) return HXE_ERROR;
  const int cancelled = static_cast<int>(PyLong_AsLong(result));
  Py_DECREF(result);
  return cancelled;
}

int hxe_request_info(hxe_engine* engine, long long request, hxe_request* out) {
  if (engine == nullptr || out == nullptr) return fail("hxe_request_info: bad arguments");
  Locked lock;
  PyObject* result = call("request", Py_BuildValue("(OL)", engine->object, request));
  if (result == nullptr) return HXE_ERROR;
  PyObject *reason = nullptr, *error = nullptr;
  const int parsed = PyArg_ParseTuple(result, "iOiiiiO", &out->state, &reason, &out->prompt_tokens,
                                      &out->generated_tokens, &out->cached_tokens,
                                      &out->preemptions, &error);
  if (parsed) {
    copy_text(out->stop_reason, sizeof out->stop_reason, reason);
    copy_text(out->error, sizeof out->error, error);
  }
  Py_DECREF(result);
  return parsed ? HXE_OK : fail(python_error());
}

int hxe_request_tokens(hxe_engine* engine, long long request, int32_t* out, int capacity) {
  if (engine == nullptr || (out == nullptr && capacity > 0)) return fail("hxe_request_tokens: bad arguments");
  Locked lock;
  PyObject* result = call("generated", Py_BuildValue("(OL)", engine->object, request));
  if (result == nullptr) return HXE_ERROR;
  const Py_ssize_t count = PyList_Size(result);
  for (Py_ssize_t i = 0; i < count && i < capacity; ++i)
    out[i] = static_cast<int32_t>(PyLong_AsLong(PyList_GET_ITEM(result, i)));
  Py_DECREF(result);
  return static_cast<int>(count);
}

int hxe_engine_stats(hxe_engine* engine, hxe_stats* out) {
  if (engine == nullptr || out == nullptr) return fail("hxe_engine_stats: bad arguments");
  Locked lock;
  PyObject* result = call("stats", Py_BuildValue("(O)", engine->object));
  if (result == nullptr) return HXE_ERROR;
  const int parsed = PyArg_ParseTuple(result, "LLLLLLLLLL", &out->iterations, &out->prefill_tokens,
                                      &out->decode_tokens, &out->finished, &out->cancelled,
                                      &out->failed, &out->preemptions, &out->steps,
                                      &out->free_pages, &out->pages);
  Py_DECREF(result);
  return parsed ? HXE_OK : fail(python_error());
}

int hxe_engine_metrics(hxe_engine* engine, hxe_metrics* out) {
  if (engine == nullptr || out == nullptr) return fail("hxe_engine_metrics: bad arguments");
  Locked lock;
  PyObject* result = call("metrics", Py_BuildValue("(O)", engine->object));
  if (result == nullptr) return HXE_ERROR;
  const int parsed = PyArg_ParseTuple(
      result, "ddddddddddd", &out->request_count, &out->finished_count, &out->failed_count,
      &out->prompt_tokens_processed, &out->generated_tokens, &out->observation_seconds,
      &out->generated_tokens_per_second, &out->time_to_first_token_p50,
      &out->time_to_first_token_p95, &out->inter_token_p50, &out->inter_token_p95);
  Py_DECREF(result);
  return parsed ? HXE_OK : fail(python_error());
}

}  // extern "C"
