// TEST INFRASTRUCTURE ONLY.  Compiles the reference's own flash-attention unit-test kernel
// (tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp, a 64 x 32 fp32 head) from where it lies in
// the reference tree and exports its launcher with C linkage, so the restatement can be checked
// against the unmodified reference program.
#include "tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp"

extern "C" int pto_ref_tflashattn_64x32(const float *q, const float *k, const float *v, float *o)
{
    LaunchTFLASHATTN(o, const_cast<float *>(q), const_cast<float *>(k), const_cast<float *>(v), nullptr);
    return 0;
}
