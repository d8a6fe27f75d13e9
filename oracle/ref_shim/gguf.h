/* Intentionally empty.
 *
 * The reference's ggml-impl.h includes "gguf.h", a header that is not part of
 * the vendored source subset.  Only two C++-only declarations use it, and the
 * C translation units compiled for the reference build never see them, so an
 * empty header on the include path is enough.  Test infrastructure only. */
