// Stand-in: the reference arithmetic only needs the mlir namespace to exist.
#pragma once
#include <cstdint>
#include <climits>
#include <cstdlib>
#include <iostream>
#include <cstddef>
#include <cmath>
#include <cassert>
#include <cstring>
#include <string>
#include <vector>
#include <algorithm>
namespace mlir {}
