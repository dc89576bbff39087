"""The reference engine itself (UCTSearch, Network, NNCache, GTP, CPUPipe: its
sources compiled unchanged as a GPU build) with CUDAPipe standing where its
OpenCLScheduler stands: the drop-in check at the level a user of the engine
sees.  Covers the engine's precision selection with its fall-back, its built-in
self-check against its own CPUPipe, the stop-the-search protocol (drain and
resume) and a move-by-move comparison of the engine on CPUPipe with the engine
on CUDAPipe.  The binary is built where the reference tree is present
(leela-zero_b200/engine/Makefile) and travels with the repository."""
import importlib.util
import os
import re

import pytest

from conftest import ROOT

ENGINE_DIR = os.path.join(ROOT, "leela-zero_b200", "engine")


def _runner():
    spec = importlib.util.spec_from_file_location("run_engine", os.path.join(ENGINE_DIR, "run_engine.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_boost_stand_ins(tmp_path):
    """The header-only stand-ins behave like the Boost calls the engine makes."""
    import subprocess
    src = tmp_path / "t.cpp"
    src.write_text(r'''
#include <boost/format.hpp>
#include <boost/algorithm/string.hpp>
#include <boost/spirit/home/x3.hpp>
#include <boost/scope_exit.hpp>
#include <boost/math/distributions/students_t.hpp>
#include <cmath>
#include <cstdio>
namespace x3 = boost::spirit::x3;
int main() {
    int bad = 0;
    bad += str(boost::format("Playouts: %d, Win: %5.2f%%, PV: %s") % 1600 % 53.217f % std::string("Q16")) != "Playouts: 1600, Win: 53.22%, PV: Q16";
    bad += boost::str(boost::format("%3d ") % 7) != "  7 ";
    bad += str(boost::format("KM[%.1f]") % 7.5f) != "KM[7.5]";
    std::string line = " 1.5 -2e-3 7  ";
    std::vector<float> w; auto it = line.cbegin();
    bad += !phrase_parse(it, line.cend(), *x3::float_, x3::space, w) || w.size() != 3 || it != line.cend();
    std::string junk = "1 2 x"; w.clear(); it = junk.cbegin();
    phrase_parse(it, junk.cend(), *x3::float_, x3::space, w);
    bad += (it == junk.cend());                       // leftover text must be visible to the caller
    int n = 0; { BOOST_SCOPE_EXIT(&n) { n = 5; } BOOST_SCOPE_EXIT_END } bad += n != 5;
    std::string s = "a\n\nb\n\nc"; boost::replace_all(s, "\n\n", "\n"); bad += s != "a\nb\nc";
    bad += !boost::algorithm::starts_with("W+Resign", "W+") || !boost::algorithm::find_first("B+Time", "Time");
    const double t = boost::math::quantile(boost::math::complement(boost::math::students_t(10), 0.025));
    bad += std::fabs(t - 2.228139) > 1e-4;             // textbook value
    const double c = boost::math::quantile(boost::math::complement(boost::math::students_t(1), 1e-5));
    bad += std::fabs(c - 31830.98862) > 1e-2;          // Cauchy: tan(pi (1/2 - alpha))
    std::printf("%d\n", bad);
    return bad;
}
''')
    exe = str(tmp_path / "t")
    subprocess.run(["g++", "-std=c++17", "-I" + os.path.join(ENGINE_DIR, "boost_shim"), str(src), "-o", exe],
                   check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout


def _engine():
    run_engine = _runner()
    if not os.path.exists(run_engine.EXE):
        pytest.skip("engine_bench not built (needs the reference tree)")
    return run_engine


TREE_BYTES = 3000000     # stops each deterministic search after roughly 700 simulations


def test_engine_with_cpupipe_behind_the_scheduler_is_repeatable():
    """The deterministic mode (one seeded search thread, searches ended by the
    tree-size limit) gives the same game twice; the comparison of two pipes
    below rests on that.  engine_check is the engine built as for the GPU, with
    the reference's CPUPipe doing the arithmetic behind CUDAPipe's queue
    (tests/cpp/engine_cpupipe_backend.cpp): no GPU needed.  The engine's own
    --cpu-only run is repeatable too, but plays another game: without a GPU
    pipe the engine draws no self-check lots from the random generator
    (src/Network.cpp:786-788), so the random symmetries differ."""
    run_engine = _engine()
    kw = dict(blocks=2, filters=32, threads=1, batch=1, gpus=1, visits=0, moves=4, seed=2082,
              deterministic=TREE_BYTES)
    a = run_engine.run(precision="single", exe=run_engine.EXE_CHECK, **kw)
    b = run_engine.run(precision="single", exe=run_engine.EXE_CHECK, **kw)
    assert a["moves"] == 4 and a["nn_evals"] > 4 * 100
    assert a["move_list"] == b["move_list"] and a["engine_playouts"] == b["engine_playouts"]
    c = run_engine.run(cpu_only=True, **kw)
    d = run_engine.run(cpu_only=True, **kw)
    assert c["pipe"] == "CPUPipe" and c["move_list"] == d["move_list"]


def test_precision_selection_and_fall_back_without_a_gpu():
    """Network::select_precision on the stand-in scheduler, with the CPUPipe
    checker as backend: auto takes the half-precision pipe without a timing run
    and checks it once against the CPU pipe; when that pipe refuses to
    initialise the engine falls back to single precision
    (src/Network.cpp:426-441)."""
    run_engine = _engine()
    kw = dict(blocks=2, filters=32, threads=2, batch=2, gpus=1, visits=30, moves=3, seed=2084,
              exe=run_engine.EXE_CHECK, precision="auto", selfchecks=2)
    ok = run_engine.run(**kw)
    assert "using fp16/half or tensor core compute support" in ok["log"]
    assert "Falling back" not in ok["log"] and ok["pipe"] == "CUDAPipe fp16x2"
    fb = run_engine.run(inject_half_init_failure=1, **kw)
    assert "Falling back to single precision" in fb["log"]
    assert fb["pipe"] == "CUDAPipe fp32" and fb["moves"] == 3 and fb["selfchecks_passed"] == 2


@pytest.mark.gpu
def test_engine_on_cudapipe_plays_the_same_game_as_on_cpupipe():
    """Same weights, same seed, one search thread, the engine's own precision
    setting "single": the engine with CUDAPipe's fp32 kernels plays the moves
    it plays with the reference's CPUPipe behind the same queue, with the same
    number of playouts (12 moves, about 700 simulations each)."""
    run_engine = _engine()
    kw = dict(blocks=2, filters=32, threads=1, batch=1, gpus=1, visits=0, moves=12, seed=2082,
              deterministic=TREE_BYTES, precision="single")
    cpu = run_engine.run(exe=run_engine.EXE_CHECK, **kw)
    gpu = run_engine.run(**kw)
    assert gpu["pipe"] == "CUDAPipe fp32" and gpu["nn_evals"] > 12 * 100
    assert gpu["move_list"] == cpu["move_list"], (gpu["move_list"], cpu["move_list"])
    assert gpu["engine_playouts"] == cpu["engine_playouts"]


@pytest.mark.gpu
@pytest.mark.parametrize("precision,pipe", [("single", "CUDAPipe fp32"), ("auto", "CUDAPipe fp16x2"),
                                            ("fp16", "CUDAPipe fp16"), ("bf16", "CUDAPipe bf16")])
def test_engine_self_check_passes(precision, pipe):
    """The engine's own comparison of its GPU pipe with its CPUPipe
    (Network::compare_net_outputs, src/Network.cpp:667-690), forced after each
    of 8 moves on a 6 x 64 network; with precision auto the engine's
    select_precision also runs it once while choosing (src/Network.cpp:426-431)."""
    run_engine = _engine()
    out = run_engine.run(blocks=6, filters=64, threads=2, batch=2, gpus=1, visits=40, moves=8,
                         precision=precision, seed=2083, selfchecks=8)
    assert out["pipe"] == pipe
    assert out["selfchecks_passed"] == 8 and out["moves"] == 8
    if precision == "auto":
        assert "using fp16/half or tensor core compute support" in out["log"]
        assert "Falling back" not in out["log"]


@pytest.mark.gpu
def test_half_precision_failure_falls_back_to_single():
    """A half-precision pipe that refuses to initialise (injected on the host)
    is replaced by the single-precision one, as the engine does for OpenCL
    (src/Network.cpp:426-441), and the game goes on."""
    run_engine = _engine()
    out = run_engine.run(blocks=2, filters=32, threads=2, batch=2, gpus=1, visits=40, moves=4,
                         precision="auto", seed=2084, selfchecks=2, inject_half_init_failure=1)
    assert "Falling back to single precision" in out["log"]
    assert out["pipe"] == "CUDAPipe fp32" and out["moves"] == 4 and out["selfchecks_passed"] == 2


@pytest.mark.gpu
def test_search_end_halts_queued_callers():
    """UCTSearch::think ends a search with drain_evals / resume_evals
    (src/UCTSearch.cpp:829-832).  Through the engine that must reach
    CUDAPipe::drain: search threads still queued for a batch leave with
    NetworkHaltException (counted by the pipe) and the next search runs."""
    run_engine = _engine()
    out = run_engine.run(blocks=2, filters=32, threads=8, batch=8, gpus=1, visits=150, moves=10,
                         precision="half", seed=2085, batching="wait")
    assert out["moves"] == 10 and out["halted"] > 0
    assert out["nn_evals"] >= 10 * 50


@pytest.mark.gpu
def test_engine_plays_on_cudapipe():
    """A short game: 4 search threads, 100 visits per move.  The engine must
    produce legal GTP moves and every evaluation must have gone through the
    pipe in batches."""
    run_engine = _engine()
    out = run_engine.run(blocks=2, filters=32, threads=4, batch=4, gpus=1, visits=100, moves=8,
                         precision="fp16", seed=2080)
    assert out["moves"] == 8 and len(out["gtp_moves"]) == 8
    assert all(re.fullmatch(r"[A-HJ-T](1[0-9]|[1-9])|pass|resign", m) for m in out["gtp_moves"])
    assert len(set(out["gtp_moves"]) - {"pass"}) >= 6        # different points: the board is being played on
    assert out["nn_evals"] >= 8 * 50                          # at least half the visits needed a fresh evaluation
    assert out["batches"] < out["nn_evals"]                   # requests were batched
    assert out.get("engine_playouts", 0) > 0                  # the engine's own statistics line was seen


@pytest.mark.gpu
def test_concurrent_games_share_the_queue():
    """Six games at once, two search threads each, one network: all games
    finish their moves and the batches are larger than one tree's two callers
    could make them."""
    run_engine = _engine()
    out = run_engine.run(blocks=2, filters=32, threads=2, batch=12, gpus=1, visits=60, moves=6,
                         precision="fp16", seed=2081, games=6, batching="eager")
    assert out["games"] == 6 and out["moves"] == 36
    assert out["nn_evals"] >= 36 * 20
    assert out["mean_batch"] > 2.0
