"""CPU oracle for the LayerNorm / RMSNorm kernels -- test infrastructure, not product code."""
