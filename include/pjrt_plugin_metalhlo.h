/*
 * pjrt_plugin_metalhlo_b200.so -- the PJRT plugin of the B200 backend.
 *
 * Replaces the reference's PJRTMetalHLO dynamic library (Sources/PJRTMetalHLO/PJRTApi.swift:15-21: `GetPjrtApi`,
 * the one symbol a PJRT host such as XLA or JAX looks up after dlopen). The returned table follows the OpenXLA PJRT
 * C API, version 0.90 (pjrt_c_api.h, which this repository does not carry; a host that loads plugins already has
 * it). Entries filled: the same set the reference fills (PJRTApi.swift:23-160), plus
 * PJRT_Executable_OptimizedProgram, PJRT_Executable_GetCompiledMemoryStats, PJRT_Buffer_UnsafePointer and
 * PJRT_Buffer_OpaqueDeviceMemoryDataPointer, which the reference answers with UNIMPLEMENTED.
 *
 * Behaviour kept from the reference: platform name "metalhlo", platform version "0.1.0"; one addressable device with
 * one memory space of kind "device"; programs arrive as StableHLO text; transfers and execution complete before the
 * call returns, so every PJRT_Event handed out is already ready; the optimisation level comes from
 * METALHLO_OPT_LEVEL (O0..O3, default O2); a serialized executable is
 * [u32 version = 1][u64 text length][StableHLO text] and loading one re-compiles the text at O2.
 */
#ifndef PJRT_PLUGIN_METALHLO_H
#define PJRT_PLUGIN_METALHLO_H

#ifdef __cplusplus
extern "C" {
#endif

struct PJRT_Api;
const struct PJRT_Api* GetPjrtApi(void);

#ifdef __cplusplus
}
#endif
#endif /* PJRT_PLUGIN_METALHLO_H */
