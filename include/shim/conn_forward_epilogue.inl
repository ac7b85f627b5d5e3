/*
 * Body fragment for ConnLayer<Device::CUDA>::forward when inferring(), replacing include/cuda/ConnLayer.h:187-216 (cuDNN
 * batch-norm inference or addBiasGpu, the preActivation_ copy, activation_->apply) after the cublasGemm call: the
 * conv epilogue on a 1x1 map with one channel per output.  training() keeps the reference's lines.
 *
 * Uses the reference's members output_, batch(), outputs(), batchNorm_, scales_, biases_, rollingMean_, rollingVar_;
 * added by the integration: pxeActivation_ (int).
 */
{
    pxe_epilogue_desc d{};
    d.x = this->output_.data();
    d.y = this->output_.data();
    d.batch = this->batch();
    d.channels = this->outputs();
    d.height = 1;
    d.width = 1;
    if (batchNorm_) {
        d.gamma = scales_.data();
        d.beta = biases_.data();
        d.mean = rollingMean_.data();
        d.var = rollingVar_.data();
        d.eps = 0.00001f;
        d.eps_mode = PXE_BN_EPS_CUDNN;
    } else {
        d.bias = biases_.data();
    }
    d.act = pxeActivation_;
    PXE_CHECK(pxe_conv_epilogue(nullptr, &d));
}
