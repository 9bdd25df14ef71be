"""TEST INFRASTRUCTURE: CPU oracle of the linear-layer path (not part of the product)."""
