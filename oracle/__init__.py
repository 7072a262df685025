"""CPU checker for the attention path.  Test infrastructure, never a product path."""
