/*
 * Body fragment for SoftmaxLayer<Device::CUDA>::forward(const V& input), replacing the cudnnSoftmaxForward call of
 * include/cuda/SoftmaxLayer.h:72-74.  pxe_softmax follows the CPU layer (include/SoftmaxLayer.h:86-99): `groups_`
 * contiguous groups per image and `temperature_`; cuDNN's channel mode is groups = 1, temperature = 1 on a 1x1
 * map.  The training() lines after it (computeLoss, cublasSasum) stay as they are -- computeLoss already calls
 * px::softmaxCrossEntropy, which the link-compatible tier provides.
 *
 * Uses the reference's members output_, batch(), inputs(), groups_, temperature_.
 */
{
    PXE_CHECK(pxe_softmax(nullptr, input.data(), this->output_.data(), this->batch(), this->inputs(), groups_, temperature_));
}
