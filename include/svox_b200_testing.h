/*
 * Test hook of libsvox_b200 -- NOT part of the stable C ABI (no counterpart in
 * the reference).  The library's own tests use it to show that two internal
 * choices change no result; a binding for the reference has no use for it and
 * it may change or disappear in any version.
 */
#ifndef SVOX_B200_TESTING_H
#define SVOX_B200_TESTING_H

#ifdef __cplusplus
extern "C" {
#endif

/* key 5: MB of gradient that one leaf-range bin of the replay backward spans
 *        (1..1024, default 32);
 * key 7: bricks below the render leaf table (1 = on, the default; 0 = off).
 * Process-wide; an index built by svoxb_render_scratch_build is invalid after
 * key 7 changes.  Unknown keys return SVOXB_ERR_OPTION. */
int svoxb_test_knob(int key, int value);

#ifdef __cplusplus
}
#endif
#endif /* SVOX_B200_TESTING_H */
