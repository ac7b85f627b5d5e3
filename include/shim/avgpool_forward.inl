/*
 * Body fragment for AvgPoolLayer<Device::CUDA>::forward(const V& input), replacing the cudnnPoolingForward call of
 * include/cuda/AvgPoolLayer.h:71-73 (global average over each channel's plane, include/AvgPoolLayer.h:66-87): no
 * pooling or tensor descriptors needed.
 *
 * Uses the reference's members output_, batch(), channels(), height(), width(), outputs().
 */
{
    PXE_CHECK(pxe_avgpool(nullptr, input.data(), 0, this->output_.data(), this->outputs(), this->batch(), this->channels(),
                          this->height(), this->width()));
}
