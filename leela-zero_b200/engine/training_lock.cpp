// Serialises the engine's training record so that several searches can run in
// one process.  UCTSearch::think ends with Training::record(...)
// (src/UCTSearch.cpp:847), which appends to a process-wide vector without a
// lock (src/Training.cpp:208, src/Training.h:103): fine for the engine's one
// search at a time, a data race for concurrent games.  The engine's sources are
// compiled as they are; the linker (--wrap) sends the search's call here, and
// this takes a mutex around the engine's own function.
#include <mutex>

class Network;
class GameState;
class UCTNode;

extern "C" {
// Training::record(Network&, GameState const&, UCTNode const&), Itanium C++ ABI name
void __real__ZN8Training6recordER7NetworkRK9GameStateRK7UCTNode(Network&, const GameState&,
                                                               const UCTNode&);
void __wrap__ZN8Training6recordER7NetworkRK9GameStateRK7UCTNode(Network& network,
                                                               const GameState& state,
                                                               const UCTNode& root) {
    static std::mutex m;
    std::lock_guard<std::mutex> lk(m);
    __real__ZN8Training6recordER7NetworkRK9GameStateRK7UCTNode(network, state, root);
}
}
