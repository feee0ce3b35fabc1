/*
 * nncp_dropin.c -- builds the reference's own command-line compressor (nncp.c, unmodified,
 * compiled from where it lies) with its Transformer model class re-pointed at the B200
 * library.  The reference source is pulled in by #include so that the adapter can use its
 * file-local types; nothing of it is copied.  Build: oracle/Makefile, target `dropin`.
 */
#include "nncp.c"

#include "trf_cuda_model.inc"

__attribute__((constructor)) static void nncp_dropin_install(void)
{
    trf_cuda_install();
}
