"""CPU oracle for sig / sig_backprop: test infrastructure, never imported by the product."""
