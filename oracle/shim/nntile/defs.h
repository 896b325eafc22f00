/* Stand-in for the header the reference's CMake generates from
 * include/nntile/defs.h.in.  CBLAS on; the CUDA switch is passed on the command
 * line by oracle/build.py so that bf16 stores round to nearest even like the
 * reference's CUDA build.  TEST INFRASTRUCTURE ONLY. */
#pragma once
#define NNTILE_USE_CBLAS
