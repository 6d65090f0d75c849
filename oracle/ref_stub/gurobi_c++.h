/* Stand-in for the commercial solver's header, which is not installed here.  The reference's
 * extraction source includes its solver header, which in turn includes this one and only needs
 * the type to be complete (a static_assert on its size).  Used ONLY to compile the reference's
 * extraction kernels, in place, into the parity-pin binary under oracle/_ref/; no solver code
 * is compiled or called. */
#pragma once
class GRBVar {
  void* p;
};
