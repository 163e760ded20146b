// Empty stand-in: the reference's src/Tensor.h includes thpp/Storage.h, but the
// CPU convolution file uses nothing from it.  TEST INFRASTRUCTURE ONLY.
#pragma once
