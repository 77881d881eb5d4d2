// Compile-time switch for the kernels' self-measurement code (role cycle counters, launch
// timelines, experiment knobs read from the environment).  The product build leaves
// HOM_DIAGNOSTICS undefined: none of that code, and none of its kernel parameters, exists
// then.  `python build.py --diagnostics` builds a second copy of the libraries with it.
#pragma once

#ifdef HOM_DIAGNOSTICS
#define HOM_DIAG(...) __VA_ARGS__
#define HOM_DIAG_ENABLED 1
#else
#define HOM_DIAG(...)
#define HOM_DIAG_ENABLED 0
#endif
