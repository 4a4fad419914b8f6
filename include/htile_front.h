/*
 * htile_front -- stand-alone C++ front end for HTile programs (text in, object model out).
 *
 * Takes the place, for the B200 target, of the reference's C++ dialect plugin loaded into mlir-opt
 * (lib/HTile/HTileDialect.cpp, lib/HTile/HTileOps.cpp: parsing and verification of the htile ops and
 * of #htile.encoding; lib/HTile/HTilePasses.cpp:52-141: the dot-transpose-to-load-order pass) and of
 * the mlir-opt round trip in src/neptune_mlir/translators/common.py:200-229.  No LLVM, no MLIR: a
 * recursive-descent reader for the subset of MLIR custom assembly that HTile programs are written in
 * (func.func, gpu.launch, scf.for/yield, arith/math element-wise ops, linalg.broadcast, tensor.empty
 * and the htile ops of include/HTile/HTileOps.td:21-217).
 *
 * Host code only; plain C ABI.  All functions are thread-safe on distinct modules.
 */
#ifndef HTILE_FRONT_H
#define HTILE_FRONT_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct htf_module htf_module;

/* Library version as major*10000 + minor*100 + patch. */
int htf_version(void);

/* Parse program text.  Returns NULL on a syntax error, unknown op, undefined SSA value or unsupported
 * type, with "line N: message (at 'snippet')" in err (always NUL-terminated when err_len > 0). */
htf_module *htf_parse(const char *text, char *err, size_t err_len);

void htf_free(htf_module *m);

/* Structural checks of the htile ops (operand counts and ranks, shapes of dot / reduce / permute /
 * load / store results, dimension_order and permutation being permutations, scf.for / scf.yield
 * agreement).  Returns 0 if the module is well formed, -1 with a message in err otherwise. */
int htf_verify(const htf_module *m, char *err, size_t err_len);

/* Run a pass pipeline written in mlir-opt syntax, e.g. the reference's
 * "builtin.module(htile-dot-transpose-to-load-order,cse,canonicalize)" (common.py:16-18).
 * htile-dot-transpose-to-load-order: transpose_a / transpose_b on an htile.dot becomes an explicit
 * htile.permute [1, 0]; a permute fed by an htile.load is folded into a load with the permuted result
 * type and a dimension_order array (post-conditions: tests/test_translators.py:250-257).  cse and
 * canonicalize are accepted and change nothing that a translator reads.  Returns 0, or -1 with err. */
int htf_run_pipeline(htf_module *m, const char *pipeline, char *err, size_t err_len);

/* The object model as JSON (functions, blocks, operations, values with ids, types as text,
 * attributes); the caller frees the string with htf_string_free. */
char *htf_to_json(const htf_module *m);

/* The module as HTile custom assembly, values renumbered %0, %1, ... in definition order. */
char *htf_print(const htf_module *m);

void htf_string_free(char *s);

#ifdef __cplusplus
}
#endif

#endif /* HTILE_FRONT_H */
