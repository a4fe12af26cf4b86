"""pi0.7 on the PaliGemma backbone (the layout of checkpoints trained before the move to Gemma-3)."""
