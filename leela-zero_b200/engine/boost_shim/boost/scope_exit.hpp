// Minimal stand-in for BOOST_SCOPE_EXIT(captures) { body } BOOST_SCOPE_EXIT_END:
// runs the body when the enclosing scope is left, also by an exception
// (src/UCTSearch.cpp:247-249).  Captures are taken by reference.
#ifndef LZB_BOOST_SHIM_SCOPE_EXIT_HPP
#define LZB_BOOST_SHIM_SCOPE_EXIT_HPP
#include <utility>

namespace lzb_shim {
template <typename F>
class scope_guard {
public:
    explicit scope_guard(F f) : m_f(std::move(f)) {}
    scope_guard(scope_guard&& o) : m_f(std::move(o.m_f)), m_active(o.m_active) { o.m_active = false; }
    ~scope_guard() { if (m_active) m_f(); }
private:
    F m_f;
    bool m_active = true;
};
template <typename F>
scope_guard<F> make_scope_guard(F f) { return scope_guard<F>(std::move(f)); }
}  // namespace lzb_shim

#define LZB_SHIM_CAT2(a, b) a##b
#define LZB_SHIM_CAT(a, b) LZB_SHIM_CAT2(a, b)
#define BOOST_SCOPE_EXIT(...) \
    auto LZB_SHIM_CAT(lzb_scope_exit_, __LINE__) = ::lzb_shim::make_scope_guard([&]()
#define BOOST_SCOPE_EXIT_END );
#endif
