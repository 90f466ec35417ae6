"""CPU oracle: test infrastructure only (see blockscaled.py). Never imported by the product package."""
