// Process-wide switches of the kernel library.
#include "common.cuh"

static int g_pdl_enabled = 0;

// Programmatic dependent launch on (1) or off (0, the default) for every kernel
// launched afterwards.  Off gives plain stream order; results are the same.
// Measured on a decode step of 6 layers at batch 8: 1.011 ms off, 1.002 ms with
// only the matrix products on, 1.19 ms with every kernel on (the early-launched
// blocks of later kernels crowd the attention kernel), so it stays off.
extern "C" void vx_set_pdl(int enabled) { g_pdl_enabled = enabled ? 1 : 0; }
extern "C" int vx_pdl_is_enabled(void) { return g_pdl_enabled; }

static int g_pdl_mask = ~0;
// Which kernel classes (VX_K_*, one bit each) are launched programmatically.
extern "C" void vx_set_pdl_mask(int mask) { g_pdl_mask = mask; }
extern "C" int vx_pdl_mask(void) { return g_pdl_mask; }
