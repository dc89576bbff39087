// Minimal stand-in for the one use of boost::math in the engine
// (src/Utils.cpp:56-63): the upper quantile of Student's t distribution,
//   quantile(complement(students_t(v), alpha)) = t with P(T > t) = alpha.
// P(T > t) = I_x(v/2, 1/2) / 2 with x = v / (v + t^2) for t > 0, where I is the
// regularised incomplete beta function (continued fraction, modified Lentz);
// t is found by bisection on a logarithmic scale.
#ifndef LZB_BOOST_SHIM_STUDENTS_T_HPP
#define LZB_BOOST_SHIM_STUDENTS_T_HPP
#include <cmath>

namespace boost {
namespace math {

struct students_t {
    double v;
    explicit students_t(double degrees) : v(degrees) {}
};
struct students_t_complement {
    students_t dist;
    double alpha;
};
inline students_t_complement complement(const students_t& d, double alpha) {
    return students_t_complement{d, alpha};
}

namespace detail {
inline double incomplete_beta(double a, double b, double x) {
    if (x <= 0.0) return 0.0;
    if (x >= 1.0) return 1.0;
    if (x > (a + 1.0) / (a + b + 2.0)) return 1.0 - incomplete_beta(b, a, 1.0 - x);
    const double lnfront = std::lgamma(a + b) - std::lgamma(a) - std::lgamma(b) + a * std::log(x) +
                           b * std::log1p(-x);
    const double tiny = 1e-300;
    double f = 1.0, c = 1.0, d = 0.0;
    for (int i = 0; i <= 400; i++) {
        const int m = i / 2;
        double num;
        if (i == 0) num = 1.0;
        else if (i % 2 == 0) num = (m * (b - m) * x) / ((a + 2.0 * m - 1.0) * (a + 2.0 * m));
        else num = -((a + m) * (a + b + m) * x) / ((a + 2.0 * m) * (a + 2.0 * m + 1.0));
        d = 1.0 + num * d;
        if (std::fabs(d) < tiny) d = tiny;
        d = 1.0 / d;
        c = 1.0 + num / c;
        if (std::fabs(c) < tiny) c = tiny;
        const double cd = c * d;
        f *= cd;
        if (std::fabs(1.0 - cd) < 1e-14) break;
    }
    return std::exp(lnfront) * (f - 1.0) / a;
}
inline double upper_tail(double v, double t) {
    return 0.5 * incomplete_beta(0.5 * v, 0.5, v / (v + t * t));
}
}  // namespace detail

inline double quantile(const students_t_complement& c) {
    const double v = c.dist.v, alpha = c.alpha;
    if (alpha >= 0.5) return 0.0;
    double lo = 1e-6, hi = 1e12;       // upper_tail is decreasing in t
    for (int i = 0; i < 200; i++) {
        const double mid = std::sqrt(lo * hi);
        if (detail::upper_tail(v, mid) > alpha) lo = mid; else hi = mid;
    }
    return std::sqrt(lo * hi);
}

}  // namespace math
}  // namespace boost
#endif
