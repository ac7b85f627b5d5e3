/*
 * Body fragment for RegionLayer<Device::CUDA>::forward(const V& input) when inferring(), replacing the device -> host
 * -> device round trip of include/cuda/RegionLayer.h:43-53 (whole input and output copied to the host, forwardCpu,
 * copied back): the transpose to per-box records, the logistic on the objectness entry and the optional softmax over
 * each box's classes (include/RegionLayer.h:271-300) run on the device.  training() keeps the reference's lines
 * (forwardCpu also computes the loss).
 *
 * Uses the reference's members output_, batch(), width(), height(), classes(), num_, coords_, softmax_.
 */
{
    PXE_CHECK(pxe_region_forward(nullptr, input.data(), this->output_.data(), this->batch(), this->width(), this->height(),
                                 num_, coords_, this->classes(), softmax_ ? 1 : 0));
}
