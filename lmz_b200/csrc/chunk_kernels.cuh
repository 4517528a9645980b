// chunk kernels (filled in below)
