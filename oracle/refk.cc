/*
 * refk -- a minimal CUDA driver-API launcher for the REFERENCE's own kernels.  Test and benchmark infrastructure: it is
 * never linked into, loaded by or shipped with the product library.
 *
 * The reference compiles each .cu file to a cubin, loads it with cuModuleLoadData and launches kernels by name with
 * cuLaunchKernelEx, PDL and cluster attributes included (crates/kernels/src/lib.rs:28-49, crates/cuda/src/lib.rs:571-664).
 * This file does the same for the cubins that oracle/Makefile builds from the reference's sources into oracle/_ref/.
 * Everything that decides WHAT is launched -- parameter structs, grids, clusters, shared-memory sizes, tensor maps,
 * weight layouts -- is restated in oracle/refkernels.py, where it can be checked on a CPU; this file only forwards it to
 * the driver.  It uses the calling thread's current context (the primary context the host framework created).
 */
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static char g_err[512];

static int fail(CUresult r, const char* what) {
    const char* name = nullptr;
    cuGetErrorName(r, &name);
    snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, name ? name : "?", (int)r);
    return (int)r > 0 ? (int)r : -1;
}

extern "C" {

const char* refk_last_error(void) { return g_err; }

/* cuModuleLoad of one cubin file. */
int refk_load(const char* path, void** module_out) {
    CUmodule m = nullptr;
    CUresult r = cuModuleLoad(&m, path);
    if (r != CUDA_SUCCESS) return fail(r, path);
    *module_out = (void*)m;
    return 0;
}

int refk_unload(void* module) {
    CUresult r = cuModuleUnload((CUmodule)module);
    return r == CUDA_SUCCESS ? 0 : fail(r, "cuModuleUnload");
}

/* Kernel by name (Kernels::get, crates/kernels/src/lib.rs:47-49). */
int refk_function(void* module, const char* name, void** fn_out) {
    CUfunction f = nullptr;
    CUresult r = cuModuleGetFunction(&f, (CUmodule)module, name);
    if (r != CUDA_SUCCESS) return fail(r, name);
    *fn_out = (void*)f;
    return 0;
}

/* Function::set_max_dynamic_smem / allow non-portable cluster sizes (crates/cuda/src/lib.rs:540-569). */
int refk_set_smem(void* fn, int bytes) {
    CUresult r = cuFuncSetAttribute((CUfunction)fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, bytes);
    return r == CUDA_SUCCESS ? 0 : fail(r, "cuFuncSetAttribute(max dynamic smem)");
}
int refk_allow_big_cluster(void* fn) {
    CUresult r = cuFuncSetAttribute((CUfunction)fn, CU_FUNC_ATTRIBUTE_NON_PORTABLE_CLUSTER_SIZE_ALLOWED, 1);
    return r == CUDA_SUCCESS ? 0 : fail(r, "cuFuncSetAttribute(non-portable cluster)");
}
int refk_func_attr(void* fn, int attr, int* value) {
    CUresult r = cuFuncGetAttribute(value, (CUfunction_attribute)attr, (CUfunction)fn);
    return r == CUDA_SUCCESS ? 0 : fail(r, "cuFuncGetAttribute");
}

/* cu::launch (crates/cuda/src/lib.rs:630-664): cuLaunchKernelEx with the programmatic-stream-serialization attribute
 * when `pdl` and a cluster dimension attribute when cx*cy*cz > 1.  `params` is the kernelParams array. */
int refk_launch(void* fn, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz, unsigned smem, unsigned cx,
                unsigned cy, unsigned cz, int pdl, void* stream, void** params) {
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = gz;
    cfg.blockDimX = bx; cfg.blockDimY = by; cfg.blockDimZ = bz;
    cfg.sharedMemBytes = smem;
    cfg.hStream = (CUstream)stream;
    CUlaunchAttribute attrs[2];
    memset(attrs, 0, sizeof(attrs));
    unsigned n = 0;
    if (pdl) {
        attrs[n].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attrs[n].value.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cx * cy * cz > 1) {
        attrs[n].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attrs[n].value.clusterDim.x = cx;
        attrs[n].value.clusterDim.y = cy;
        attrs[n].value.clusterDim.z = cz;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    CUresult r = cuLaunchKernelEx(&cfg, (CUfunction)fn, params, nullptr);
    return r == CUDA_SUCCESS ? 0 : fail(r, "cuLaunchKernelEx");
}

/* The reference's tensor-map constructors (crates/cuda/src/lib.rs:694-808), encoded into a 128-byte host buffer that the
 * caller uploads (the kernels read their maps from global memory).  All: interleave none, OOB fill none. */
static int encode(void* out, CUtensorMapDataType dt, unsigned rank, uint64_t base, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box, CUtensorMapSwizzle sw, CUtensorMapL2promotion l2, const char* what) {
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    CUtensorMap m;
    CUresult r = cuTensorMapEncodeTiled(&m, dt, rank, (void*)base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, l2,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(r, what);
    memcpy(out, &m, sizeof(m));
    return 0;
}

/* tensor_map_u8_sw128 (lib.rs:742-763): dims {cols, rows}, row stride `stride` bytes, box {128, box_rows}, 128-byte swizzle. */
int refk_tmap_u8_sw128(void* out, uint64_t base, uint64_t cols, uint64_t rows, uint64_t stride, uint32_t box_rows) {
    cuuint64_t dims[2] = {cols, rows}, strides[1] = {stride};
    cuuint32_t box[2] = {128, box_rows};
    return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "tensor_map_u8_sw128");
}

/* tensor_map_fp4_rows (lib.rs:765-786): dims {16, rows, 4}, strides {64, 16}, box {16, box_rows, 4}, no swizzle. */
int refk_tmap_fp4_rows(void* out, uint64_t base, uint64_t rows, uint32_t box_rows) {
    cuuint64_t dims[3] = {16, rows, 4}, strides[2] = {64, 16};
    cuuint32_t box[3] = {16, box_rows, 4};
    return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "tensor_map_fp4_rows");
}

/* tensor_map_fp4_unpack_strided (lib.rs:694-715): 4-bit elements widened by TMA; dims {d0, d1, d2}, strides {d0/2, d2_stride},
 * box {128, box_rows, 1}, 128-byte swizzle. */
int refk_tmap_fp4_unpack_strided(void* out, uint64_t base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d2_stride, uint32_t box_rows) {
    cuuint64_t dims[3] = {d0, d1, d2}, strides[2] = {d0 / 2, d2_stride};
    cuuint32_t box[3] = {128, box_rows, 1};
    return encode(out, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "tensor_map_fp4_unpack_strided");
}

}  /* extern "C" */
