"""The reference engine itself (UCTSearch, Network, NNCache, GTP: its sources
compiled unchanged) playing on top of CUDAPipe: the drop-in check at the level
a user of the engine sees.  The binary is built where the reference tree is
present (leela-zero_b200/engine/Makefile) and travels with the repository."""
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


@pytest.mark.gpu
def test_engine_plays_on_cudapipe():
    """A short game: 4 search threads, 100 visits per move.  The engine must
    produce legal GTP moves and every evaluation must have gone through the
    pipe in batches."""
    run_engine = _runner()
    if not os.path.exists(run_engine.EXE):
        pytest.skip("engine_bench not built (needs the reference tree)")
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
    run_engine = _runner()
    if not os.path.exists(run_engine.EXE):
        pytest.skip("engine_bench not built (needs the reference tree)")
    out = run_engine.run(blocks=2, filters=32, threads=2, batch=12, gpus=1, visits=60, moves=6,
                         precision="fp16", seed=2081, games=6, batching="eager")
    assert out["games"] == 6 and out["moves"] == 36
    assert out["nn_evals"] >= 36 * 20
    assert out["mean_batch"] > 2.0
