// Definitions of the opaque handle types of the C ABI (declared in include/mcb.h), shared by the
// translation units that implement entry points on them.
#pragma once
#include "autograd.h"

struct mcb_var {
    mcbag::Var v;
};
struct mcb_adam {
    mcbag::AdamOpt opt;
};
struct mcb_scaler {
    mcbag::Scaler *s;
};
struct mcb_arena {
    mcbag::Arena *a;
};
struct mcb_model {
    mcbag::Model *m;
};
