// Minimal stand-in for the boost string algorithms the engine calls:
// replace_all, find_first (used as a truth value), starts_with, trim, icontains.
#ifndef LZB_BOOST_SHIM_ALGORITHM_STRING_HPP
#define LZB_BOOST_SHIM_ALGORITHM_STRING_HPP
#include <algorithm>
#include <cctype>
#include <string>

namespace boost {
namespace algorithm {

inline void replace_all(std::string& s, const std::string& from, const std::string& to) {
    if (from.empty()) return;
    size_t pos = 0;
    while ((pos = s.find(from, pos)) != std::string::npos) {
        s.replace(pos, from.size(), to);
        pos += to.size();
    }
}
struct find_result {
    bool found;
    explicit operator bool() const { return found; }
};
inline find_result find_first(const std::string& s, const std::string& what) {
    return find_result{s.find(what) != std::string::npos};
}
inline bool starts_with(const std::string& s, const std::string& prefix) {
    return s.compare(0, prefix.size(), prefix) == 0;
}
inline void trim(std::string& s) {
    auto not_space = [](unsigned char c) { return !std::isspace(c); };
    s.erase(s.begin(), std::find_if(s.begin(), s.end(), not_space));
    s.erase(std::find_if(s.rbegin(), s.rend(), not_space).base(), s.end());
}
inline bool icontains(const std::string& s, const std::string& what) {
    auto lower = [](std::string v) {
        std::transform(v.begin(), v.end(), v.begin(), [](unsigned char c) { return std::tolower(c); });
        return v;
    };
    return lower(s).find(lower(what)) != std::string::npos;
}

}  // namespace algorithm
using algorithm::icontains;
using algorithm::replace_all;
using algorithm::starts_with;
using algorithm::trim;
}  // namespace boost
#endif
