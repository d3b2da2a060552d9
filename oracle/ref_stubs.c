/* ref_stubs.c - link-time stand-ins for the reference's Q4_K linear launcher.
 *
 * TEST INFRASTRUCTURE ONLY. oracle/_ref/libq3ref.so is the reference's own
 * src/q3_forward.cu compiled where it lies; that file also contains the full
 * forward runtime, which calls five quantised-GEMM entry points from other
 * reference files. The attention primitives never reach them, so they are
 * stubbed here to fail instead of dragging the GEMM closure into the build.
 */
#include <stdbool.h>
#include <stddef.h>

bool q3_q4_linear_bind_geometry(void) { return false; }
bool q3_cuda_q4k_linear(void) { return false; }
bool q3_cuda_q4k_linear_init(void) { return false; }
bool q3_cuda_q4k_linear_set_workspace(void) { return false; }
size_t q3_cuda_q4k_linear_workspace_bytes(void) { return 0; }
