/* clpeak C ABI -- the outermost drop-in boundary.
 *
 * The six symbols below are the complete native bridge the clpeak GUI binds by
 * name over Dart FFI (reference: src/ffi/clpeak_ffi.h:28-105, bound in
 * app/lib/src/ffi/clpeak_bindings.dart:38-50).  libclpeak_ffi.so of this
 * repository exports exactly these, with the same signatures, ownership rules
 * and return codes; the "CUDA" backend behind them is the sm_100a backend.
 *
 * String ownership: `char *` results are malloc'd UTF-8 and must be released
 * with clpeak_free_string(); `const char *` results are static.
 */
#ifndef CLPEAK_FFI_H
#define CLPEAK_FFI_H

#if defined(_WIN32)
#define CLPEAK_FFI_EXPORT __declspec(dllexport)
#else
#define CLPEAK_FFI_EXPORT __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces clpeak_version (src/ffi/clpeak_ffi.h:28).  Static string. */
CLPEAK_FFI_EXPORT const char *clpeak_version(void);

/* Replaces clpeak_copy_backend_catalog_json (clpeak_ffi.h:30-34): the device
 * catalog of every backend in this library as
 *   {"backends":[{"name","available","platforms":[{"index","name",
 *     "devices":[{"index","name","type",...}]}]}]}                            */
CLPEAK_FFI_EXPORT char *clpeak_copy_backend_catalog_json(void);

/* Replaces clpeak_free_string (clpeak_ffi.h:36). */
CLPEAK_FFI_EXPORT void clpeak_free_string(char *s);

/* Every run event arrives as one malloc'd JSON document whose ownership passes
 * to the callee (clpeak_ffi.h:40-65).  Kinds ("t"): backend_begin, device,
 * test_begin, metric, test_skipped, test_end, device_end, backend_end, note,
 * done.  Callbacks fire on the thread that called clpeak_launch(). */
typedef void (*ClpeakEventCallback)(void *user_data, char *event_json);

#define CLPEAK_RUN_OK         0
#define CLPEAK_RUN_BAD_ARGS  (-1)
#define CLPEAK_RUN_CANCELLED (-2)
#define CLPEAK_RUN_BUSY      (-3)

/* Replaces clpeak_launch (clpeak_ffi.h:75-84).  Blocking; argv[0] is the program
 * name and the rest follows the CLI grammar; --xml-file / --json-file /
 * --csv-file are honoured at the end of the run (also after a cancel).  A final
 * {"t":"done","status":..,"cancelled":..} event is always emitted, except when
 * the call returns CLPEAK_RUN_BUSY.  Never calls exit(). */
CLPEAK_FFI_EXPORT int clpeak_launch(int argc, const char **argv, ClpeakEventCallback on_event, void *user_data);

/* Replaces clpeak_request_cancel (clpeak_ffi.h:86-92).  Any thread; observed at
 * test boundaries; reset by the next clpeak_launch(). */
CLPEAK_FFI_EXPORT void clpeak_request_cancel(void);

/* Replaces clpeak_load_result_file_json (clpeak_ffi.h:94-105): a saved XML /
 * JSON / CSV result file re-serialised as the saveJson document; NULL when the
 * file is unreadable, rejected or empty. */
CLPEAK_FFI_EXPORT char *clpeak_load_result_file_json(const char *path);

#ifdef __cplusplus
}
#endif
#endif /* CLPEAK_FFI_H */
