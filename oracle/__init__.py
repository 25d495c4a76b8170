"""CPU oracle for the grouped-affine matmul path.  Test infrastructure only:
the product package never imports this."""
