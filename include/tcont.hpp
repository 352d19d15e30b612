// Drop-in name for the reference's public header: callers written against TconT's
// include/tcont.hpp (its bench_tccg harness, for one) compile against this file unchanged.
#pragma once
#include "tcont_b200/tcont_api.hpp"
