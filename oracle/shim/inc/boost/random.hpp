// Test infrastructure (oracle build only): the two boost::random names the reference's dropout bridge
// mentions, expressed with <random>.  The convolution path never draws from them.
#ifndef CCT_ORACLE_SHIM_BOOST_RANDOM_HPP
#define CCT_ORACLE_SHIM_BOOST_RANDOM_HPP
#include <random>
namespace boost {
template <class T>
struct bernoulli_distribution {
  T prob;
  explicit bernoulli_distribution(T p = T(0.5)) : prob(p) {}
};
template <class Engine, class Dist>
struct variate_generator {
  Engine eng;
  Dist dist;
  variate_generator(Engine e, Dist d) : eng(e), dist(d) {}
  float operator()() { return std::bernoulli_distribution(dist.prob)(eng) ? 1.0f : 0.0f; }
};
}  // namespace boost
#endif
