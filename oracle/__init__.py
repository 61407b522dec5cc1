"""CPU oracle for the AMO-BQ hot path.  Test infrastructure, never a product path."""
