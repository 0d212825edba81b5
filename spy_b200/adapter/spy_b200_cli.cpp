// Command-line driver for the reference's token loop on either backend: the counterpart of the reference's `spy`
// executable (app/cli/src/cli.cpp:12-49, app/cli/include/cli.h:60-129) for runs that need no tokenizer - the prompt is
// given as token ids - with the sm_100a backend selectable the way the reference selects backends
// (BackendFactory::init_backend("gpu:b200", ...), backend/interface/include/backend/backend.h:109-117).
//
//   spy_b200_cli -m model.gguf --token-ids 1,15043,3186 [-n 32] [-c 512] [--backend cpu:default|gpu:b200] [--plan 0|1] [-t threads]
//
// It links the library that holds the reference's own sources plus the adapter (the token loop itself is the
// reference's: graph builder, scheduler, loader, greedy sampler) and prints the generated ids and the timing lines of
// PerformanceTimer::print_timing (util/include/util/timer.h:66-79).
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

extern "C" int spy_ref_generate(const char *gguf_path, const int32_t *prompt, int n_prompt, int n_predict, int num_context,
                                int num_thread, int warmup, int32_t *out_ids, float *out_logits, double *step_ms);

static void usage(const char *argv0) {
    std::fprintf(stderr, "usage: %s -m model.gguf --token-ids id,id,... [-n num_predict] [-c num_context] [--backend cpu:default|gpu:b200] "
                         "[--plan 0|1] [-t num_thread] [--no-warmup]\n", argv0);
}

int main(int argc, char **argv) {
    std::string model, backend = "gpu:b200", ids_arg;
    int num_predict = 32, num_context = 512, num_thread = 8, plan = 1, warmup = 1;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> const char * { if (i + 1 >= argc) { usage(argv[0]); std::exit(2); } return argv[++i]; };
        if (a == "-m" || a == "--model") { model = next(); }
        else if (a == "--token-ids") { ids_arg = next(); }
        else if (a == "-n" || a == "--num-predict") { num_predict = std::atoi(next()); }
        else if (a == "-c" || a == "--num-context") { num_context = std::atoi(next()); }
        else if (a == "-t" || a == "--num-thread") { num_thread = std::atoi(next()); }
        else if (a == "--backend") { backend = next(); }
        else if (a == "--plan") { plan = std::atoi(next()); }
        else if (a == "--no-warmup") { warmup = 0; }
        else { usage(argv[0]); return 2; }
    }
    std::vector<int32_t> prompt;
    for (size_t pos = 0; pos < ids_arg.size();) {
        size_t end = ids_arg.find(',', pos);
        if (end == std::string::npos) { end = ids_arg.size(); }
        prompt.push_back((int32_t)std::atoi(ids_arg.substr(pos, end - pos).c_str()));
        pos = end + 1;
    }
    if (model.empty() || prompt.empty() || num_predict < 1) { usage(argv[0]); return 2; }
    int thread_arg = num_thread;
    if (backend == "gpu:b200" || backend == "gpu:default") { thread_arg = plan ? -2 : -1; }
    else if (backend != "cpu:default") { std::fprintf(stderr, "unknown backend %s\n", backend.c_str()); return 2; }

    std::vector<int32_t> ids(num_predict);
    std::vector<double>  step_ms(num_predict);
    const auto t0 = std::chrono::steady_clock::now();
    const int n_vocab = spy_ref_generate(model.c_str(), prompt.data(), (int)prompt.size(), num_predict, num_context, thread_arg, warmup,
                                         ids.data(), nullptr, step_ms.data());
    const auto t1 = std::chrono::steady_clock::now();
    if (n_vocab < 0) { std::fprintf(stderr, "generation failed (%d)%s\n", n_vocab, n_vocab == -2 ? ": this build has no device backend" : ""); return 1; }
    std::printf("token ids:");
    for (int id : ids) { std::printf(" %d", id); }
    std::printf("\n");
    double decode_ms = 0;
    for (int i = 1; i < num_predict; ++i) { decode_ms += step_ms[i]; }
    const double total_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    // the lines of PerformanceTimer::print_timing; loading, graph building and the warm-up step are what the loop's own timers leave out
    std::printf("[Performance Timer] model loading: %16zu ms\n", (size_t)(total_ms - decode_ms - step_ms[0]));
    std::printf("[Performance Timer] prefill stage: %16zu ms, %g token/s\n", (size_t)step_ms[0], (float)(prompt.size() * 1000) / (float)step_ms[0]);
    std::printf("[Performance Timer] decode stage:  %16zu ms, %g token/s\n", (size_t)decode_ms, num_predict > 1 ? (float)((num_predict - 1) * 1000) / (float)decode_ms : 0.f);
    return 0;
}
