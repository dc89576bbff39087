// Minimal stand-in for boost::format, enough for the engine's six call sites
// ("%3d ", "%.1f", "Playouts: %d, Win: %5.2f%%, PV: %s", "move %d, %c => %s\n%s").
// Written for building the leela-zero engine where Boost is not installed;
// printf-style conversion of one argument per '%' directive, in order.
#ifndef LZB_BOOST_SHIM_FORMAT_HPP
#define LZB_BOOST_SHIM_FORMAT_HPP
#include <cstdio>
#include <string>
#include <type_traits>

namespace boost {

class format {
public:
    explicit format(const std::string& f) : m_fmt(f) {}

    template <typename T>
    typename std::enable_if<std::is_arithmetic<T>::value, format&>::type operator%(const T& v) {
        const std::string spec = next_spec();
        const char conv = spec.empty() ? 's' : spec.back();
        char buf[128];
        if (conv == 'd' || conv == 'i' || conv == 'u' || conv == 'x') {
            std::string s2 = spec.substr(0, spec.size() - 1) + "ll" + conv;
            std::snprintf(buf, sizeof(buf), s2.c_str(), static_cast<long long>(v));
        } else if (conv == 'c') {
            std::snprintf(buf, sizeof(buf), spec.c_str(), static_cast<int>(v));
        } else if (conv == 's') {
            std::snprintf(buf, sizeof(buf), "%g", static_cast<double>(v));
        } else {
            std::snprintf(buf, sizeof(buf), spec.c_str(), static_cast<double>(v));
        }
        m_out += buf;
        return *this;
    }
    format& operator%(const std::string& v) {
        next_spec();
        m_out += v;
        return *this;
    }
    format& operator%(const char* v) { return *this % std::string(v); }

    std::string str() const {
        format copy(*this);
        copy.flush_literal();
        return copy.m_out;
    }

private:
    // Copies literal text up to the next directive into the output and returns
    // that directive ("%5.2f"), handling "%%".
    std::string next_spec() {
        while (m_pos < m_fmt.size()) {
            if (m_fmt[m_pos] != '%') {
                m_out += m_fmt[m_pos++];
            } else if (m_pos + 1 < m_fmt.size() && m_fmt[m_pos + 1] == '%') {
                m_out += '%';
                m_pos += 2;
            } else {
                size_t end = m_pos + 1;
                while (end < m_fmt.size() && !std::isalpha(static_cast<unsigned char>(m_fmt[end]))) end++;
                std::string spec = m_fmt.substr(m_pos, end - m_pos + 1);
                m_pos = end + 1;
                return spec;
            }
        }
        return std::string();
    }
    void flush_literal() {
        while (m_pos < m_fmt.size()) {
            if (m_fmt[m_pos] == '%' && m_pos + 1 < m_fmt.size() && m_fmt[m_pos + 1] == '%') {
                m_out += '%';
                m_pos += 2;
            } else {
                m_out += m_fmt[m_pos++];
            }
        }
    }
    std::string m_fmt, m_out;
    size_t m_pos = 0;
};

inline std::string str(const format& f) { return f.str(); }

}  // namespace boost
#endif
