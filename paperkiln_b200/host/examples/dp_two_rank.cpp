// Data-parallel training without Python: one process per GPU, the checkpointed training step of
// libmicrotorch and the in-library gradient exchange (mt_dp_*, NCCL through libpk's collective
// group). What a C++ trainer such as the reference's tools/mtstudio.cpp (its loop at :448-518)
// would link against.
//
//   dp_two_rank [world] [steps]        (world GPUs of this machine, default 2; default 3 steps)
//
// The parent forks `world` ranks before any CUDA call. Rank 0 draws the communicator id and
// publishes it in a temporary file; every rank builds the same small Llama (same seed), takes its
// slice of each global batch, scales its loss by 1 / world, and all-reduces the gradients of each
// block while the previous block is being recomputed. After every step the ranks' losses are
// printed; with identical weights and summed gradients the weights stay identical on all ranks,
// which rank 0 checks at the end against a checksum every rank writes.
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "mt_capi.h"

#define MT(call)                                                                      \
    do {                                                                              \
        if ((call) != 0) {                                                            \
            std::fprintf(stderr, "rank %d: %s failed: %s\n", rank, #call, mt_last_error()); \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

static bool read_file(const std::string& path, void* dst, size_t n, double timeout_s) {
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        if (FILE* f = std::fopen(path.c_str(), "rb")) {
            const size_t got = std::fread(dst, 1, n, f);
            std::fclose(f);
            if (got == n) return true;
        }
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) return false;
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
}
static bool write_file(const std::string& path, const void* src, size_t n) {
    const std::string tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) return false;
    const size_t put = std::fwrite(src, 1, n, f);
    std::fclose(f);
    return put == n && std::rename(tmp.c_str(), path.c_str()) == 0;
}

static int run_rank(int rank, int world, int steps, const std::string& dir) {
    MT(mt_init(rank, /*fp32*/ 0));
    void* model = nullptr;
    MT(mt_model_create("family=llama;vocab=512;d=128;layers=3;heads=4;kv_heads=2;dff=256;nctx=64;rope_all=1;seed=3;ckpt=1", &model));
    MT(mt_model_set_adamw(model, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f));
    unsigned char id[128];
    if (rank == 0) {
        MT(mt_dp_unique_id(id, sizeof(id)));
        if (!write_file(dir + "/id", id, sizeof(id))) return 1;
    } else if (!read_file(dir + "/id", id, sizeof(id), 60.0)) {
        std::fprintf(stderr, "rank %d: no communicator id\n", rank);
        return 1;
    }
    MT(mt_dp_init(model, id, rank, world, 0));
    MT(mt_dp_set_timeout(model, 60.0));
    const int B = 8, S = 64, per = B / world;
    std::mt19937 rng(5);   // every rank draws the same global stream and takes its slice
    for (int step = 0; step < steps; ++step) {
        std::vector<int32_t> stream(B * S + 1);
        for (auto& t : stream) t = static_cast<int32_t>(rng() % 512);
        const int32_t* ids = stream.data() + rank * per * S;
        float loss = 0.0f;
        MT(mt_model_step(model, ids, ids + 1, per * S, S, 1.0f / world, 1, &loss));
        MT(mt_dp_finish(model));       // remaining ranges; the compute stream waits for the transfers
        MT(mt_dp_wait_host(model));    // a rank that died would surface here as an error, not a hang
        MT(mt_model_optimizer_step(model));
        std::printf("rank %d step %d loss %.6f\n", rank, step, loss);
        std::fflush(stdout);
    }
    // identical weights on every rank: checksum of the first parameter
    int64_t rows = 0, cols = 0;
    char name[128];
    MT(mt_model_param_info(model, 0, name, sizeof(name), &rows, &cols));
    std::vector<float> p(static_cast<size_t>(rows * cols));
    MT(mt_model_param_get(model, 0, p.data()));
    double sum = 0.0;
    for (float v : p) sum += v;
    if (!write_file(dir + "/sum." + std::to_string(rank), &sum, sizeof(sum))) return 1;
    int rc = 0;
    if (rank == 0) {
        for (int r = 1; r < world; ++r) {
            double other = 0.0;
            if (!read_file(dir + "/sum." + std::to_string(r), &other, sizeof(other), 60.0) || other != sum) {
                std::fprintf(stderr, "weights of rank %d differ from rank 0 (%.17g vs %.17g)\n", r, other, sum);
                rc = 1;
            }
        }
        std::printf("%s: %d ranks, %d steps, parameter checksum %.9g on every rank\n", rc ? "MISMATCH" : "OK", world, steps, sum);
    }
    MT(mt_dp_destroy(model));
    MT(mt_model_destroy(model));
    return rc;
}

int main(int argc, char** argv) {
    const int world = argc > 1 ? std::atoi(argv[1]) : 2;
    const int steps = argc > 2 ? std::atoi(argv[2]) : 3;
    if (world < 1 || world > 8 || 8 % world != 0 || steps < 1) {
        std::fprintf(stderr, "usage: dp_two_rank [world in {1,2,4,8}] [steps >= 1]\n");
        return 2;
    }
    char tmpl[] = "/tmp/pk_dp_XXXXXX";
    if (!mkdtemp(tmpl)) return 2;
    const std::string dir = tmpl;
    std::vector<pid_t> kids;
    for (int r = 0; r < world; ++r) {
        const pid_t pid = fork();
        if (pid == 0) {
            const int rc = run_rank(r, world, steps, dir);
            std::fflush(stdout);
            std::fflush(stderr);
            _exit(rc);
        }
        if (pid < 0) return 2;
        kids.push_back(pid);
    }
    int rc = 0;
    for (pid_t k : kids) {
        int st = 0;
        waitpid(k, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) rc = 1;
    }
    const std::string rm = "rm -rf '" + dir + "'";
    if (std::system(rm.c_str()) != 0) rc = rc ? rc : 0;
    return rc;
}
