// placeholder, replaced by the tcgen05 implementation
#include "common.cuh"
XB_API int xb_tc_supported(const XbConvGeom*, int) { return 0; }
XB_API int xb_conv_fprop_tc(const float*, const float*, const float*, float*, float*, const XbConvGeom*, int, int*, cudaStream_t) { return -XB_BAD_ARG; }
XB_API int xb_conv_dgrad_tc(const float*, const float*, float*, const XbConvGeom*, int, int*, cudaStream_t) { return -XB_BAD_ARG; }
XB_API int xb_conv_wgrad_tc(const float*, const float*, float*, const XbConvGeom*, int*, cudaStream_t) { return -XB_BAD_ARG; }
