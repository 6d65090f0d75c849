/* Stand-in for a TBB header that is not installed here; the reference's solver header
 * includes it but the extraction kernels compiled into the parity-pin binary use nothing of it. */
#pragma once
