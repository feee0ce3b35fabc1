/* nncp-metal: the command-line tool (main of src/metal/nncp_metal.c:1229 in the reference);
   everything lives in libnncp_host.so (nncpm_main, include/nncp_metal_frontend.h). */
#include "nncp_metal_frontend.h"

int main(int argc, char **argv) { return nncpm_main(argc, argv); }
