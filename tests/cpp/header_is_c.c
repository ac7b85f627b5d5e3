/* The public headers are plain C: this file is compiled with -std=c99 -pedantic -Werror. */
#include "pxe.h"
#include "pxe_plan.h"

int header_is_c(void)
{
    pxe_epilogue_desc d;
    pxe_epilogue_nhwc_desc n;
    pxe_layer_desc l;
    pxe_step s;
    pxe_detection det;
    (void)d; (void)n; (void)l; (void)s;
    return (int)sizeof(det);
}
