// train_bloom: fine-tune driver over the words machine, one process per GPU.
//
// Plays the part of the reference's driver (blackriver/train_bloom.cpp: BloomInput produces ids and
// masks, BloomAttentions loads the words scripts and runs them) for one pipeline stage per rank.
// Differences that follow from the model living in HBM: there is no feeder rank (every rank reads or
// generates the same token ids; the first stage gathers the embeddings on the device), no weight
// streaming, and the stage's script is generated for the model size
// (python -m blackriver_b200.emit_stage) instead of being fixed to two stages of BLOOMZ-7b.
//
// Ranks come from the environment (RANK, WORLD_SIZE, LOCAL_RANK, as set by torchrun, mpirun
// wrappers or a shell loop); the NCCL id travels through a file that rank 0 writes (--id-file).
//
// Per step: every micro-batch forward (receive from the previous stage, run, send on), then every
// micro-batch backward, then the two holders of the tied embedding table sum their gradients, then Adam.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include <unistd.h>

#include "common.hpp"
#include "context.hpp"
#include "dag.hpp"
#include "nn.hpp"
#include "tensortype.hpp"

namespace {

struct Options {
    std::string script, data, id_file;      // id_file default: a name shared by the processes of one launch (same parent)
    int layers = -1;          // decoder layers of THIS stage (hash tables = layers + 1)
    int steps = 3, micro = 1, batch = 2, tokens = 128, vocab = 250880, min_len = 1;
    uint64_t seed = 3;
    double lr = 1e-4, loss_scale = 1024.0;
    int verbose = 0;
};

void usage() {
    std::fprintf(stderr,
                 "usage: train_bloom --script STAGE.words --layers N --batch B --tokens T [--micro M] [--steps S]\n"
                 "                   [--vocab V] [--min-len L] [--seed S] [--lr LR] [--loss-scale X]\n"
                 "                   [--data PREFIX] [--id-file PATH] [--verbose]\n"
                 "  STAGE.words   script of this rank's stage (python -m blackriver_b200.emit_stage prints the command)\n"
                 "  --data PREFIX raw int32 files PREFIX.ids.bin, PREFIX.mask.bin [micro, batch, tokens] and\n"
                 "                PREFIX.lens.bin [micro, batch]; without it seeded random ids with right padding\n"
                 "  --id-file     where rank 0 publishes the NCCL id (default /tmp/train_bloom.<parent pid>.ncclid)\n"
                 "  environment   RANK, WORLD_SIZE, LOCAL_RANK (default 0, 1, 0)\n");
}

bool parse(int argc, char** argv, Options& o) {
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        auto next = [&]() -> const char* {
            if (i + 1 >= argc) {
                std::fprintf(stderr, "missing value after %s\n", a.c_str());
                std::exit(2);
            }
            return argv[++i];
        };
        if (a == "--script") o.script = next();
        else if (a == "--data") o.data = next();
        else if (a == "--id-file") o.id_file = next();
        else if (a == "--layers") o.layers = std::atoi(next());
        else if (a == "--steps") o.steps = std::atoi(next());
        else if (a == "--micro") o.micro = std::atoi(next());
        else if (a == "--batch") o.batch = std::atoi(next());
        else if (a == "--tokens") o.tokens = std::atoi(next());
        else if (a == "--vocab") o.vocab = std::atoi(next());
        else if (a == "--min-len") o.min_len = std::atoi(next());
        else if (a == "--seed") o.seed = std::strtoull(next(), nullptr, 10);
        else if (a == "--lr") o.lr = std::atof(next());
        else if (a == "--loss-scale") o.loss_scale = std::atof(next());
        else if (a == "--verbose") o.verbose = 1;
        else if (a == "--help" || a == "-h") return false;
        else {
            std::fprintf(stderr, "unknown argument %s\n", a.c_str());
            return false;
        }
    }
    return !o.script.empty() && o.layers >= 0 && o.steps > 0 && o.micro > 0 && o.batch > 0 && o.tokens > 0;
}

int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v ? std::atoi(v) : fallback;
}

std::string read_text(const std::string& path) {
    std::ifstream f(path);
    br_assert(f.good(), ("cannot open " + path).c_str());
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

std::vector<int> read_ints(const std::string& path, size_t count) {
    std::ifstream f(path, std::ios::binary);
    br_assert(f.good(), ("cannot open " + path).c_str());
    std::vector<int> v(count);
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)(count * sizeof(int)));
    br_assert((size_t)f.gcount() == count * sizeof(int), ("short read from " + path).c_str());
    return v;
}

uint64_t splitmix(uint64_t& s) {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct MicroBatches {
    std::vector<int> ids, mask, lens;      // [micro][batch][tokens], same, [micro][batch]
};

// Same bytes on every rank: a pure function of the options.
MicroBatches make_data(const Options& o) {
    MicroBatches d;
    const size_t bt = (size_t)o.batch * o.tokens, n = (size_t)o.micro * bt;
    if (!o.data.empty()) {
        d.ids = read_ints(o.data + ".ids.bin", n);
        d.mask = read_ints(o.data + ".mask.bin", n);
        d.lens = read_ints(o.data + ".lens.bin", (size_t)o.micro * o.batch);
        return d;
    }
    d.ids.resize(n);
    d.mask.resize(n);
    d.lens.resize((size_t)o.micro * o.batch);
    uint64_t s = o.seed;
    const int lo = o.min_len < 1 ? 1 : (o.min_len > o.tokens ? o.tokens : o.min_len);
    for (int m = 0; m < o.micro; m++)
        for (int b = 0; b < o.batch; b++) {
            const int len = lo + (int)(splitmix(s) % (uint64_t)(o.tokens - lo + 1));
            d.lens[(size_t)m * o.batch + b] = len;
            for (int t = 0; t < o.tokens; t++) {
                const size_t i = ((size_t)m * o.batch + b) * o.tokens + t;
                const int id = (int)(splitmix(s) % (uint64_t)o.vocab);
                d.mask[i] = t < len ? 1 : 0;
                d.ids[i] = t < len ? id : 3;      // right padding with the pad id of the reference's fixtures
            }
        }
    return d;
}

// ids [batch, tokens], mask [batch, tokens] and lens [batch] of micro-batch m, packed in the order of the stage
// script's device tensor "inp"
std::vector<int> packed_inputs(const Options& o, const MicroBatches& d, int m) {
    const size_t bt = (size_t)o.batch * o.tokens;
    std::vector<int> p;
    p.reserve(2 * bt + o.batch);
    p.insert(p.end(), d.ids.begin() + (size_t)m * bt, d.ids.begin() + (size_t)(m + 1) * bt);
    p.insert(p.end(), d.mask.begin() + (size_t)m * bt, d.mask.begin() + (size_t)(m + 1) * bt);
    p.insert(p.end(), d.lens.begin() + (size_t)m * o.batch, d.lens.begin() + (size_t)(m + 1) * o.batch);
    return p;
}

}  // namespace

int main(int argc, char** argv) {
    Options o;
    if (!parse(argc, argv, o)) {
        usage();
        return 2;
    }
    const int rank = env_int("RANK", 0), world = env_int("WORLD_SIZE", 1), local = env_int("LOCAL_RANK", rank);
    if (o.id_file.empty()) o.id_file = "/tmp/train_bloom." + std::to_string((long)getppid()) + ".ncclid";
    try {
        br::ComputingContext::boot(local);
        if (world > 1) br::CollectiveContext::boot_from_file(rank, world, o.id_file);

        const bool first = rank == 0, last = rank == world - 1;
        const int n_slots = world > 1 ? o.micro : 1;
        br::Enviroment env((size_t)o.layers + 1);
        br::load_nn_words(env);
        env.execute(read_text(o.script));
        env.execute("build_model init_model zero_grads");
        {
            std::stringstream ss;
            ss << o.loss_scale << " op.loss_scale " << o.verbose << " op.verbose";
            env.execute(ss.str());
        }
        std::vector<br::DaG*> fwd, bwd;          // one program per micro-batch: its slot, and the cell of "loss_all" it fills
        for (int m = 0; m < o.micro; m++) {
            std::stringstream f, b;
            f << "slot_" << (m % n_slots) << " stage_forward";
            b << "slot_" << (m % n_slots) << " \"loss@" << m << "\" stage_backward_async";
            fwd.push_back(env.build(f.str()));
            bwd.push_back(env.build(b.str()));
        }
        br::DaG* begin = env.build("zero_grads 1 op.accumulate");
        br::DaG* sync = env.build("op.sync");
        br::DaG* status = env.build("op.kernel_status");

        const MicroBatches data = make_data(o);
        const size_t bt = (size_t)o.batch * o.tokens;
        // the packed inputs live (unchanged) for the whole run, so the queued copies may read them at any later time
        std::vector<std::vector<int>> packed;
        for (int m = 0; m < o.micro; m++) packed.push_back(packed_inputs(o, data, m));
        auto feed = [&](int m) {
            env.change(0);
            br::tensor_t t = env.hash().find_tensor("inp");
            br_assert(t->is_cuda() && t->bytes() == packed[m].size() * sizeof(int), "unexpected input tensor \"inp\"");
            BR_CUDA_CHECK(cudaMemcpyAsync(t->data(), packed[m].data(), t->bytes(), cudaMemcpyHostToDevice, br::ComputingContext::cuda_stream));
        };
        std::vector<float> losses((size_t)o.micro);

        for (int step = 1; step <= o.steps; step++) {
            env.run(sync);
            const auto t0 = std::chrono::steady_clock::now();
            env.run(begin);
            if (world == 1) {
                for (int m = 0; m < o.micro; m++) {
                    feed(m);
                    env.run(fwd[m]);
                    env.run(bwd[m]);
                }
            } else {
                for (int m = 0; m < o.micro; m++) {
                    feed(m);
                    env.run(fwd[m]);
                }
                for (int m = 0; m < o.micro; m++) {
                    feed(m);
                    env.run(bwd[m]);
                }
            }
            // the one wait of the step: no update is applied on top of a tensor-core kernel that gave up a wait
            env.run(status);
            const int code = (int)env.stack().pop_number();
            br_assert(code < 256, "the previous optimizer step met non-finite gradients: lower --loss-scale");
            br_assert(code == 0, "a tensor-core kernel gave up a bounded wait; the optimizer step was not applied");
            double loss_sum = 0.0;
            int loss_n = 0;
            if (last) {
                env.change(0);
                br::tensor_t t = env.hash().find_tensor("loss_all");
                BR_CUDA_CHECK(cudaMemcpy(losses.data(), t->data(), losses.size() * sizeof(float), cudaMemcpyDeviceToHost));
                for (float v : losses) loss_sum += v;
                loss_n = o.micro;
            }
            if (world > 1 && (first || last)) {      // the two holders of the tied table sum their gradients
                std::stringstream ss;
                ss << (first ? world - 1 : 0) << " sync_tied_grads";
                env.execute(ss.str());
            }
            {
                // gradients were summed over the micro-batches and carry the loss scale: Adam divides both out
                std::stringstream ss;
                ss.precision(17);
                ss << "0 op.accumulate " << o.lr << " " << step << " " << 1.0 / (o.loss_scale * o.micro) << " optimizer_step";
                env.execute(ss.str());
            }
            env.run(sync);
            const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            if (loss_n > 0)
                std::printf("step %d rank %d loss %.6f  %.1f ms  %.0f tokens/s\n", step, rank, loss_sum / loss_n, ms,
                            (double)o.micro * bt / (ms * 1e-3));
            else
                std::printf("step %d rank %d  %.1f ms\n", step, rank, ms);
            std::fflush(stdout);
        }

        for (auto* p : fwd) delete p;
        for (auto* p : bwd) delete p;
        delete begin;
        delete sync;
        delete status;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "train_bloom rank %d: %s\n", rank, e.what());
        return 1;
    }
    if (world > 1) br::CollectiveContext::shutdown();
    br::ComputingContext::shutdown();
    return 0;
}
