// Stand-in for the Kokkos mdspan header that the reference fetches at build time
// (include/firefly/tensor_view.h:6-8 includes <mdspan/mdspan.hpp> and uses namespace Kokkos).
// The CUDA toolkit's libcu++ carries the same interface.
#pragma once
#include <cuda/std/mdspan>
namespace Kokkos = cuda::std;
