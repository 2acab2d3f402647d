/* helix_b200/engine.h: the engine for C and C++ callers.
 *
 * The reference exposes its runtime to C++ as a class with submit / run_iteration / cancel /
 * request / metrics / stats (include/helix/runtime/cpu_engine.hpp:70-98).  This header gives a
 * C++ program the same surface over THIS engine: `helix_b200::Engine` below, a thin class over
 * the C functions `hxe_*` of `libhelix_b200_engine.so`.
 *
 * What is behind it.  The engine's host side (configuration, weight loading, the cache
 * manager, the scheduler, the step function, CUDA graphs) is written once, in the Python
 * package `helix_runtime_b200`; the library hosts that package in an interpreter it embeds and
 * keeps one engine object per handle.  A C++ caller therefore runs exactly the scheduler, the
 * cache and the kernels that a Python caller runs: there is no second copy of any of them.
 * The process needs the Python that has `torch` installed: the library starts the interpreter
 * named by the environment variable HELIX_B200_PYTHON (else `python3` on PATH), so that its
 * site-packages are found, and finds the package next to itself.  A process that already runs
 * Python (the library loaded from a Python program) is used as it is.
 *
 * Threads: calls may come from any thread; they are serialised by the interpreter's lock.
 * Errors: the C functions return 0 or a negative code and leave a message for
 * hxe_last_error() (per thread); the C++ class throws helix_b200::Error with that message.
 *
 * Build (CUDA is not needed to compile a caller):
 *   g++ -std=c++17 caller.cpp -I include -L <dir of the library> -lhelix_b200_engine \
 *       -Wl,-rpath,<dir of the library>
 * The library itself is built by `python -m helix_runtime_b200.csrc.build` (printed last).
 */
#ifndef HELIX_B200_ENGINE_H
#define HELIX_B200_ENGINE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hxe_engine hxe_engine;

/* a zeroed hxe_config asks for every default */
typedef struct hxe_config {
  const char* dtype;             /* "bfloat16" (NULL: that) or "float32" */
  int device;                    /* CUDA device index */
  int page_size;                 /* keys per cache page (0: 16) */
  int num_pages;                 /* 0: enough for max_running_requests full contexts */
  int max_running_requests;      /* 0: 8 */
  int max_tokens_per_iteration;  /* 0: 2048 */
  int max_prefill_chunk;         /* 0: prompts are cut by the token budget only */
  int prefix_cache_entries;      /* > 0: prompts share the pages of a common beginning */
  int no_cuda_graphs;            /* 1: do not replay decode steps as CUDA graphs */
  int no_lookahead;              /* 1: do not queue the next decode step ahead */
} hxe_config;

enum hxe_state { HXE_WAITING = 0, HXE_PREFILL = 1, HXE_DECODING = 2, HXE_FINISHED = 3,
                 HXE_CANCELLED = 4, HXE_FAILED = 5 };

typedef struct hxe_iteration {
  int idle;                      /* nothing could be planned */
  int scheduled_tokens, prefill_tokens, decode_tokens, sampled, retired, preempted, kv_limited;
} hxe_iteration;

typedef struct hxe_request {
  int state;                     /* hxe_state */
  char stop_reason[32];          /* max_new_tokens, eos_token, context_limit, cancelled, failed */
  int prompt_tokens, generated_tokens, cached_tokens, preemptions;
  char error[256];
} hxe_request;

typedef struct hxe_stats {
  long long iterations, prefill_tokens, decode_tokens, finished, cancelled, failed, preemptions,
      steps, free_pages, pages;
} hxe_stats;

typedef struct hxe_metrics {
  double request_count, finished_count, failed_count, prompt_tokens_processed, generated_tokens,
      observation_seconds, generated_tokens_per_second, time_to_first_token_p50,
      time_to_first_token_p95, inter_token_p50, inter_token_p95;
} hxe_metrics;

#define HXE_OK 0
#define HXE_ERROR (-1)          /* see hxe_last_error() */

const char* hxe_last_error(void);
/* model: a folder with config.json and safetensors, or a Helix model file (MODEL.helix) */
int hxe_engine_create(const char* model, const hxe_config* config, hxe_engine** out);
void hxe_engine_destroy(hxe_engine* engine);
/* returns the request's id (>= 0) or HXE_ERROR; eos_token < 0: none */
long long hxe_submit(hxe_engine* engine, const int32_t* prompt, int prompt_tokens,
                     int max_new_tokens, int eos_token, float temperature, uint64_t seed);
int hxe_run_iteration(hxe_engine* engine, hxe_iteration* out);
/* max_iterations <= 0: until every request has ended */
int hxe_run_until_done(hxe_engine* engine, long long max_iterations, long long* iterations);
/* 1: cancelled, 0: the request had ended already, HXE_ERROR: no such request */
int hxe_cancel(hxe_engine* engine, long long request);
int hxe_request_info(hxe_engine* engine, long long request, hxe_request* out);
/* copies at most `capacity` generated token ids; returns how many the request has */
int hxe_request_tokens(hxe_engine* engine, long long request, int32_t* out, int capacity);
int hxe_engine_stats(hxe_engine* engine, hxe_stats* out);
int hxe_engine_metrics(hxe_engine* engine, hxe_metrics* out);

#ifdef __cplusplus
}  /* extern "C" */

#include <stdexcept>
#include <string>
#include <vector>

namespace helix_b200 {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct EngineConfig {
  std::string dtype = "bfloat16";
  int device = 0;
  int page_size = 16;
  int num_pages = 0;
  int max_running_requests = 8;
  int max_tokens_per_iteration = 2048;
  int max_prefill_chunk = 0;
  int prefix_cache_entries = 0;
  bool cuda_graphs = true;
  bool lookahead = true;
};

struct SubmitOptions {
  int max_new_tokens = 32;
  int eos_token = -1;
  float temperature = 0.0f;
  uint64_t seed = 0;
};

struct RequestView {
  hxe_state state;
  std::string stop_reason, error;
  int prompt_tokens, cached_tokens, preemptions;
  std::vector<int32_t> generated_tokens;
};

class Engine {
 public:
  Engine(const std::string& model, const EngineConfig& config = EngineConfig()) {
    hxe_config c{config.dtype.c_str(), config.device, config.page_size, config.num_pages,
                 config.max_running_requests, config.max_tokens_per_iteration,
                 config.max_prefill_chunk, config.prefix_cache_entries,
                 config.cuda_graphs ? 0 : 1, config.lookahead ? 0 : 1};
    check(hxe_engine_create(model.c_str(), &c, &handle_));
  }
  ~Engine() { hxe_engine_destroy(handle_); }
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  long long submit(const std::vector<int32_t>& prompt, const SubmitOptions& options = {}) {
    const long long id = hxe_submit(handle_, prompt.data(), static_cast<int>(prompt.size()),
                                    options.max_new_tokens, options.eos_token,
                                    options.temperature, options.seed);
    if (id < 0) throw Error(hxe_last_error());
    return id;
  }
  hxe_iteration run_iteration() {
    hxe_iteration result{};
    check(hxe_run_iteration(handle_, &result));
    return result;
  }
  long long run_until_done(long long max_iterations = 0) {
    long long iterations = 0;
    check(hxe_run_until_done(handle_, max_iterations, &iterations));
    return iterations;
  }
  bool cancel(long long request) {
    const int cancelled = hxe_cancel(handle_, request);
    if (cancelled < 0) throw Error(hxe_last_error());
    return cancelled == 1;
  }
  RequestView request(long long request) {
    hxe_request info{};
    check(hxe_request_info(handle_, request, &info));
    RequestView view{static_cast<hxe_state>(info.state), info.stop_reason, info.error,
                     info.prompt_tokens, info.cached_tokens, info.preemptions, {}};
    view.generated_tokens.resize(static_cast<size_t>(info.generated_tokens));
    const int count = hxe_request_tokens(handle_, request, view.generated_tokens.data(),
                                         info.generated_tokens);
    if (count < 0) throw Error(hxe_last_error());
    view.generated_tokens.resize(static_cast<size_t>(count < info.generated_tokens
                                                         ? count : info.generated_tokens));
    return view;
  }
  hxe_stats stats() {
    hxe_stats result{};
    check(hxe_engine_stats(handle_, &result));
    return result;
  }
  hxe_metrics metrics() {
    hxe_metrics result{};
    check(hxe_engine_metrics(handle_, &result));
    return result;
  }

 private:
  static void check(int code) {
    if (code != HXE_OK) throw Error(hxe_last_error());
  }
  hxe_engine* handle_ = nullptr;
};

}  // namespace helix_b200
#endif  /* __cplusplus */
#endif  /* HELIX_B200_ENGINE_H */
