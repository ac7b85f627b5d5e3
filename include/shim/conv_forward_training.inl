/*
 * Body fragment for ConvLayer<Device::CUDA>::forward when training(), replacing include/cuda/ConvLayer.h:284-307 for
 * layers with batchNorm_: x_.copy(output_), cudnnBatchNormalizationForwardTraining, preActivation_.copy(output_) and
 * activation_->apply(output_) become one call.  The convolution writes into x_ instead of output_ (pass x_.data() as
 * its y), so the saved input needs no copy; preActivation_ receives the normalised tensor and output_ its activation.
 * #include it right after the PX_CHECK_CUDNN that follows cudnnConvolutionForward.
 *
 * Uses the reference's members x_, preActivation_, output_, batch(), outHeight(), outWidth(), filters_, scales_,
 * biases_, rollingMean_, rollingVar_, mean_, var_; and, added by the integration: pxeActivation_ (int) and
 * pxeBnWorkspace_ (a PxCudaVectorT<char> of pxe_batchnorm_workspace_bytes(batch, filters, outHeight, outWidth) bytes,
 * allocated in setup()).  mean_ / var_ receive the batch mean and 1 / sqrt(var + eps), which is what the cuDNN call
 * stored there and what conv_backward_batchnorm.inl reads back.
 */
{
    pxe_bn_train_desc d{};
    d.x = x_.data();
    d.y = this->preActivation_.data();
    d.y_act = this->output_.data();
    d.act = pxeActivation_;
    d.batch = this->batch();
    d.channels = filters_;
    d.height = this->outHeight();
    d.width = this->outWidth();
    d.gamma = scales_.data();
    d.beta = biases_.data();
    d.running_mean = rollingMean_.data();
    d.running_var = rollingVar_.data();
    d.exp_avg_factor = 0.01f;
    d.eps = 0.00001f;
    d.eps_mode = PXE_BN_EPS_CUDNN;
    d.save_mean = mean_.data();
    d.save_scale = var_.data();
    d.workspace = pxeBnWorkspace_.data();
    d.workspace_bytes = pxeBnWorkspace_.size();
    PXE_CHECK(pxe_batchnorm_forward_training(nullptr, &d));
}
