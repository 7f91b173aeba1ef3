"""CPU oracle of the matmul hot path: test infrastructure, never a product path."""
