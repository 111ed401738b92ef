// intentionally empty: included by the reference CPU GEMM but nothing from it is used
