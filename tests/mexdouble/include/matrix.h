/* matrix.h -- part of the MEX stand-in (test infrastructure): everything is declared in mex.h. */
#include "mex.h"
