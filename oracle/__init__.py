"""TEST INFRASTRUCTURE -- CPU checkers for hodu_b200; never imported by the product."""
