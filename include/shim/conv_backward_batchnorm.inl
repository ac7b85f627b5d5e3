/*
 * Body fragment for ConvLayer<Device::CUDA>::backward, replacing include/cuda/ConvLayer.h:324-335 (the batchNorm_
 * branch: cudnnBatchNormalizationBackward into xNorm_, then delta_.copy(xNorm_)): the gradient is written over
 * delta_ itself, scaleUpdates_ and biasUpdates_ are added to as betaParam = 1 did.  It follows
 * activation_->gradient(preActivation_, delta_), as in the reference.
 *
 * Uses the reference's members x_, delta_, batch(), outHeight(), outWidth(), filters_, scales_, scaleUpdates_,
 * biasUpdates_, mean_, var_; and pxeBnWorkspace_ (see conv_forward_training.inl).
 */
{
    pxe_bn_backward_desc d{};
    d.x = x_.data();
    d.dy = this->delta_.data();
    d.dx = this->delta_.data();
    d.batch = this->batch();
    d.channels = filters_;
    d.height = this->outHeight();
    d.width = this->outWidth();
    d.gamma = scales_.data();
    d.dgamma = scaleUpdates_.data();
    d.dbeta = biasUpdates_.data();
    d.save_mean = mean_.data();
    d.save_scale = var_.data();
    d.eps = 0.00001f;
    d.eps_mode = PXE_BN_EPS_CUDNN;
    d.workspace = pxeBnWorkspace_.data();
    d.workspace_bytes = pxeBnWorkspace_.size();
    PXE_CHECK(pxe_batchnorm_backward(nullptr, &d));
}
