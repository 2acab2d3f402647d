// A C++ caller of the engine: generate tokens greedily from a model and print them.
//   generate_tiny MODEL DTYPE MAX_NEW_TOKENS TOKEN [TOKEN ...]
// Prints the three lines of the command line tool, then one line of engine statistics.
#include "helix_b200/engine.h"

#include <cstdio>
#include <cstdlib>
#include <vector>

int main(int argc, char** argv) {
  if (argc < 5) return 2;
  try {
    helix_b200::EngineConfig config;
    config.dtype = argv[2];
    config.page_size = 8;
    config.max_running_requests = 2;
    helix_b200::Engine engine(argv[1], config);
    std::vector<int32_t> prompt;
    for (int i = 4; i < argc; ++i) prompt.push_back(std::atoi(argv[i]));
    helix_b200::SubmitOptions options;
    options.max_new_tokens = std::atoi(argv[3]);
    const long long id = engine.submit(prompt, options);
    const long long second = engine.submit({prompt[0], prompt[1]}, options);   // runs beside it
    engine.cancel(second);
    const long long iterations = engine.run_until_done();
    const helix_b200::RequestView view = engine.request(id);
    std::printf("generated_token_ids:");
    for (int32_t token : view.generated_tokens) std::printf(" %d", token);
    std::printf("\nstop_reason: %s\ncached_token_count: %d\n", view.stop_reason.c_str(),
                view.cached_tokens);
    const hxe_stats stats = engine.stats();
    std::printf("iterations=%lld finished=%lld cancelled=%lld free_pages=%lld pages=%lld state=%d\n",
                iterations, stats.finished, stats.cancelled, stats.free_pages, stats.pages,
                static_cast<int>(engine.request(second).state));
    return view.state == HXE_FINISHED ? 0 : 1;
  } catch (const helix_b200::Error& error) {
    std::fprintf(stderr, "generate_tiny: %s\n", error.what());
    return 1;
  }
}
