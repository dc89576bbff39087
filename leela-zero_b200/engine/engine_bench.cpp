// engine_bench: the leela-zero engine (its own UCTSearch, Network, NNCache, GTP)
// playing moves on top of CUDAPipe, to measure NN evaluations/s and playouts/s
// end to end.  Set-up follows the engine's own start-up (src/Leela.cpp:504-519)
// and its --benchmark settings (src/Leela.cpp:467-479); moves are requested
// through GTP::execute("genmove ...") (src/GTP.cpp:623-690).
//
//
// With --games N (N > 1) it plays N games at once in this one process: every
// game has its own GameState and UCTSearch (src/UCTSearch.h:113-114) with
// --threads search threads, all games share one Network and therefore one
// CUDAPipe queue, so that batches form across games (N x T callers) instead of
// inside one tree.  Self-play settings as autogtp uses them (root noise, moves
// drawn in proportion to visits for the first 30 moves) keep the games apart.
// The engine has one process-wide piece of state a search writes to, the
// training record (src/UCTSearch.cpp:847, src/Training.h:103); its call is
// serialised at link time (training_lock.cpp), the engine's sources stay as
// they are.
//
//   engine_bench --weights FILE [--threads T] [--batch B] [--gpus G] [--visits V]
//                [--moves M] [--games N] [--batching eager|wait]
//                [--precision auto|single|half|fp32|fp16|fp16x2|bf16|...]
//                [--cpu-only] [--selfchecks K] [--deterministic BYTES]
//                [--inject-half-init-failure N] [--verbose]
//
// --precision auto/single/half are the engine's own settings (cfg_precision,
// src/GTP.h:103-107); a mode name selects half (or single for fp32) and the
// arithmetic behind it.  --cpu-only is the engine's --cpu-only (cfg_cpu_only,
// src/Network.cpp:579-581): the reference's CPUPipe instead of the GPU.
// --selfchecks K forces the engine's built-in comparison of the GPU pipe with
// its CPU pipe (src/Network.cpp:781-791) after each of the first K moves; a
// mismatch ends the program like it ends the engine.
// --deterministic BYTES makes a game repeatable so that two pipes can be
// compared move by move: one search thread with a fixed random seed, no visit
// limit, each search stopped by the tree-size limit BYTES
// (cfg_max_tree_size, src/UCTSearch.cpp:645), which the search thread itself
// checks after every simulation (the visit limit is polled by the main thread
// every 10 ms, src/UCTSearch.cpp:797-823, so it stops at a different count on
// every run).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "config.h"

#include "CUDAPipe.h"
#include "GTP.h"
#include "GameState.h"
#include "Network.h"
#include "Random.h"
#include "ThreadPool.h"
#include "UCTSearch.h"
#include "Utils.h"
#include "Zobrist.h"
#include "cuda_scheduler.h"

namespace {
// The network of the many-games mode.  Every search ends with drain_evals /
// resume_evals (src/UCTSearch.cpp:829-832), which stops ALL evaluations of the
// network: right for the engine's one search at a time, wrong when other games
// are in the middle of their searches on the same network (their search
// threads would leave and those searches would never finish).  Both calls are
// virtual in the engine (src/Network.h:114-117); here they do nothing, and the
// threads of a finished search return when their current batch does.
class SharedNetwork : public Network {
public:
    void drain_evals() override {}
    void resume_evals() override {}
};

// N games at once on one shared network; returns the number of moves played.
int play_games(Network& network, int games, int moves) {
    std::vector<std::unique_ptr<GameState>> states;
    std::vector<std::unique_ptr<UCTSearch>> searches;
    for (int g = 0; g < games; g++) {
        states.emplace_back(new GameState());
        states.back()->init_game(BOARD_SIZE, KOMI);
        states.back()->set_timecontrol(0, 1, 0, 0);
        searches.emplace_back(new UCTSearch(*states.back(), network));
    }
    std::atomic<int> played{0};
    std::vector<std::thread> players;
    for (int g = 0; g < games; g++) {
        players.emplace_back([&, g] {
            Random::get_Rng().seedrandom(cfg_rng_seed + 1000 * (g + 1));
            GameState& game = *states[g];
            for (int m = 0; m < moves && game.get_passes() < 2; m++) {
                const int color = game.get_to_move();
                const int move = searches[g]->think(color);
                game.play_move(color, move);
                played++;
            }
        });
    }
    for (auto& t : players) t.join();
    return played.load();
}
}  // namespace

int main(int argc, char** argv) {
    std::string weights, precision = "auto", move_list;
    int threads = 8, batch = 8, ngpus = 1, visits = 1600, moves = 50, games = 1, selfchecks = 0;
    long long deterministic_bytes = 0;
    bool verbose = false, cpu_only = false;
    for (int i = 1; i < argc; i++) {
        const std::string k = argv[i];
        if (k == "--verbose") { verbose = true; continue; }
        if (k == "--cpu-only") { cpu_only = true; continue; }
        if (i + 1 >= argc) { std::fprintf(stderr, "missing value for %s\n", k.c_str()); return 2; }
        const std::string v = argv[++i];
        if (k == "--weights") weights = v;
        else if (k == "--threads") threads = std::atoi(v.c_str());
        else if (k == "--batch") batch = std::atoi(v.c_str());
        else if (k == "--gpus") ngpus = std::atoi(v.c_str());
        else if (k == "--visits") visits = std::atoi(v.c_str());
        else if (k == "--moves") moves = std::atoi(v.c_str());
        else if (k == "--games") games = std::atoi(v.c_str());
        else if (k == "--selfchecks") selfchecks = std::atoi(v.c_str());
        else if (k == "--deterministic") deterministic_bytes = std::atoll(v.c_str());
        else if (k == "--inject-half-init-failure") lzb_engine::fail_half_init = std::atoi(v.c_str());
        else if (k == "--batching") lzb_engine::eager = (v == "eager");
        else if (k == "--precision") precision = v;
        else { std::fprintf(stderr, "unknown option %s\n", k.c_str()); return 2; }
    }
    if (weights.empty()) { std::fprintf(stderr, "--weights is required\n"); return 2; }
    if (games < 1 || threads < 1) { std::fprintf(stderr, "bad --games/--threads\n"); return 2; }

    GTP::setup_default_parameters();
    if (precision == "auto") cfg_precision = precision_t::AUTO;
    else if (precision == "single") cfg_precision = precision_t::SINGLE;
    else if (precision == "half") cfg_precision = precision_t::HALF;
    else {
        bool ok = false;
        const auto mode = lzb_engine::precision_from_name(precision.c_str(), &ok);
        if (!ok) { std::fprintf(stderr, "unknown precision %s\n", precision.c_str()); return 2; }
        if (mode == CUDAPipe::Precision::FP32) cfg_precision = precision_t::SINGLE;
        else { cfg_precision = precision_t::HALF; lzb_engine::half_mode = mode; }
    }
    cfg_cpu_only = cpu_only;
    cfg_gpus.clear();
    for (int g = 0; g < ngpus; g++) cfg_gpus.push_back(g);
    cfg_gtp_mode = true;
    cfg_num_threads = threads;
    cfg_batch_size = batch;
    cfg_max_visits = visits;
    cfg_allow_pondering = false;
    cfg_noise = false;
    cfg_random_cnt = 0;
    cfg_rng_seed = 1;
    cfg_timemanage = TimeManagement::OFF;
    cfg_resignpct = 0;
    cfg_quiet = !verbose;
    cfg_weightsfile = weights;
    if (deterministic_bytes > 0) {
        if (games != 1) { std::fprintf(stderr, "--deterministic plays one game\n"); return 2; }
        threads = 1;
        cfg_num_threads = 1;
        cfg_max_visits = UCTSearch::UNLIMITED_PLAYOUTS;
        cfg_max_playouts = UCTSearch::UNLIMITED_PLAYOUTS;
    }
    if (games > 1) {
        cfg_noise = true;          // autogtp's self-play options: -n, -m 30
        cfg_random_cnt = 30;
        lzb_engine::callers = games * threads;
    }

    setbuf(stdout, nullptr);
    thread_pool.initialize(static_cast<size_t>(cfg_num_threads) * games);
    auto rng = std::make_unique<Random>(5489);
    Zobrist::init_zobrist(*rng);
    Random::get_Rng().seedrandom(cfg_rng_seed);
    Utils::create_z_table();
    if (deterministic_bytes > 0) {
        // The pool's one thread draws the random symmetries of the search
        // (src/Network.cpp:776); its generator is otherwise seeded from the
        // thread id (src/Random.cpp:46-51), which differs from run to run.
        Utils::ThreadGroup tg(thread_pool);
        tg.add_task([] { Random::get_Rng().seedrandom(12345); });
        tg.wait_all();
    }
    std::unique_ptr<Network> network(games > 1 ? new SharedNetwork : new Network);
    Network* net = network.get();
    try {
        // the cache is sized from the playout limit (src/Network.cpp:578-587); N games share it
        const auto playouts = std::min(cfg_max_playouts, cfg_max_visits) * games;
        network->initialize(playouts, cfg_weightsfile);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "network initialisation failed: %s\n", e.what());
        return 3;
    }
    const CUDAPipe* pipe = lzb_engine::last_pipe;
    static const char* const mode_names[] = {"fp32", "fp16", "bf16", "fp16-winograd", "bf16-winograd",
                                             "fp16x2", "fp16x3", "bf16x3"};
    const std::string pipe_name = cpu_only || !pipe ? "CPUPipe"
        : std::string("CUDAPipe ") + mode_names[static_cast<int>(pipe->precision())];
    auto game = std::make_unique<GameState>();
    if (games == 1) {
        GTP::initialize(std::move(network));
        game->init_game(BOARD_SIZE, KOMI);
        game->set_timecontrol(0, 1, 0, 0);   // infinite time, as --benchmark does
    }
    // after GTP::initialize, which sets the memory limits (src/GTP.cpp:395-412)
    if (deterministic_bytes > 0) cfg_max_tree_size = static_cast<size_t>(deterministic_bytes);

    const auto evals0 = lzb_engine::evals.load();
    const auto t0 = std::chrono::steady_clock::now();
    int played = 0, checked = 0;
    try {
        if (games > 1) {
            played = play_games(*network, games, moves);
        } else {
            for (int m = 0; m < moves; m++) {
                GTP::execute(*game, (m % 2 == 0) ? "genmove b" : "genmove w");
                played++;
                move_list += (m ? " " : "") + game->move_to_text(game->get_last_move());
                if (checked < selfchecks) {
                    // throws "OpenCL self-check mismatch." when the pipes differ by more than 0.2
                    net->get_output(game.get(), Network::Ensemble::RANDOM_SYMMETRY, -1, false, false,
                                    true);
                    checked++;
                }
                if (game->get_passes() >= 2) break;
            }
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "engine failed: %s\n", e.what());
        return 4;
    }
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    const auto evals = lzb_engine::evals.load() - evals0;
    const auto s = pipe && !cpu_only ? pipe->stats() : CUDAPipe::Stats();
    std::printf("\n{\"pipe\": \"%s\", \"games\": %d, \"moves\": %d, \"seconds\": %.3f, \"visits_per_move\": %d, "
                "\"threads\": %d, \"batch\": %d, \"batching\": \"%s\", \"gpus\": %d, \"nn_evals\": %llu, "
                "\"nn_evals_per_s\": %.1f, \"visits_per_s\": %.1f, \"batches\": %zu, \"mean_batch\": %.2f, "
                "\"timeouts\": %zu, \"halted\": %zu, \"selfchecks_passed\": %d, \"move_list\": \"%s\"}\n",
                pipe_name.c_str(), games, played, sec, visits, threads, batch,
                lzb_engine::eager ? "eager" : "wait", ngpus, evals, evals / sec,
                double(played) * visits / sec, s.batches,
                s.batches ? double(s.positions) / s.batches : 0.0, s.timeouts, s.halted, checked,
                move_list.c_str());
    return 0;
}
