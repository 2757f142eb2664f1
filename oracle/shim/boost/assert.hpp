// Stand-in for <boost/assert.hpp> (Boost is not installed): the reference only uses the two assert macros.
#pragma once
#include <cassert>
#define BOOST_ASSERT(expr) assert(expr)
#define BOOST_ASSERT_MSG(expr, msg) assert((expr) && (msg))
