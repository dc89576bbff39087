// Minimal stand-in for the one Spirit X3 expression the engine uses:
//   phrase_parse(first, last, *x3::float_, x3::space, std::vector<float>&)
// i.e. "zero or more floats separated by white space" (src/Network.cpp:273-276).
// `first` is advanced past everything consumed, trailing white space included.
#ifndef LZB_BOOST_SHIM_SPIRIT_X3_HPP
#define LZB_BOOST_SHIM_SPIRIT_X3_HPP
#include <cctype>
#include <cstdlib>
#include <string>
#include <vector>

namespace boost {
namespace spirit {
namespace x3 {

struct float_parser {};
struct many_floats {};
struct space_parser {};
static const float_parser float_{};
static const space_parser space{};
inline many_floats operator*(const float_parser&) { return many_floats{}; }

template <typename Iterator>
bool phrase_parse(Iterator& first, Iterator last, many_floats, space_parser, std::vector<float>& out) {
    const std::string text(first, last);
    const char* p = text.c_str();
    const char* const begin = p;
    while (true) {
        while (*p && std::isspace(static_cast<unsigned char>(*p))) p++;
        if (!*p) break;
        char* end = nullptr;
        const float v = std::strtof(p, &end);
        if (end == p) break;            // not a number: stop here, the caller sees the leftover
        out.push_back(v);
        p = end;
    }
    first += (p - begin);
    return true;
}

}  // namespace x3
}  // namespace spirit
}  // namespace boost
#endif
