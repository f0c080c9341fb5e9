"""CPU oracle for the quantized-matmul path: TEST INFRASTRUCTURE, never imported by the product."""
