/* Prints sizeof and a few offsetof values of every descriptor of include/pxe.h, so that the ctypes mirrors in
 * pixienn_b200/capi.py can be held to what the C compiler lays out. */
#include <stddef.h>
#include <stdio.h>

#include "pxe.h"
#include "pxe_plan.h"
#include "pxe_debug.h"

#define SIZE(t) printf(#t " %zu\n", sizeof(t))
#define OFF(t, f) printf(#t "." #f " %zu\n", offsetof(t, f))

int main(void)
{
    SIZE(pxe_detection);
    SIZE(pxe_epilogue_desc); OFF(pxe_epilogue_desc, bias); OFF(pxe_epilogue_desc, y_pool); OFF(pxe_epilogue_desc, folded_a);
    SIZE(pxe_epilogue_nhwc_desc);
    SIZE(pxe_yolo_decode_desc); OFF(pxe_yolo_decode_desc, anchors); OFF(pxe_yolo_decode_desc, head_channels_last);
    SIZE(pxe_centernet_decode_desc);
    SIZE(pxe_yolo_loss_desc);
    SIZE(pxe_bn_train_desc); OFF(pxe_bn_train_desc, save_mean); OFF(pxe_bn_train_desc, workspace_bytes);
    SIZE(pxe_bn_backward_desc); OFF(pxe_bn_backward_desc, save_scale);
    SIZE(pxe_layer_desc);
    SIZE(pxe_step);
    SIZE(pxe_bounds_report); OFF(pxe_bounds_report, address); OFF(pxe_bounds_report, file);
    return 0;
}
