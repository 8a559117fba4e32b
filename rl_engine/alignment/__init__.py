from rl_engine.alignment.model_wrappers import PolicyModelWrapper, ReferenceModelWrapper, extract_logits

__all__ = ["PolicyModelWrapper", "ReferenceModelWrapper", "extract_logits"]
