"""CPU checkers for the CUDA library. Test infrastructure only; never imported by the product."""
