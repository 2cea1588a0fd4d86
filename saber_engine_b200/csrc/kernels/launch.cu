// Process-wide switch of programmatic dependent launch (see launch.cuh).
#include "launch.cuh"

namespace saber {
static int g_pdl = 1;
int pdl_enabled() { return g_pdl; }
}  // namespace saber

extern "C" void saber_set_pdl(int on) { saber::g_pdl = on; }
extern "C" int saber_get_pdl() { return saber::g_pdl; }
