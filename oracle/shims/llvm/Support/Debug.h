// Stand-in for llvm/Support/Debug.h: debug macros compile to nothing.
#pragma once
#include "llvm/Support/raw_ostream.h"
#define LLVM_DEBUG(X) do { } while (0)
#define DEBUG_WITH_TYPE(TYPE, X) do { } while (0)
