// The opaque handle of the C ABI.
#pragma once
#include "context.h"

struct cfhe_context {
  cfhe::Context c;
};
