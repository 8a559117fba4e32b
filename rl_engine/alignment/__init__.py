from rl_engine.alignment.advantages import gae_advantages, kl_shaped_rewards, value_loss, whiten
from rl_engine.alignment.model_wrappers import PolicyModelWrapper, ReferenceModelWrapper, extract_logits

__all__ = ["PolicyModelWrapper", "ReferenceModelWrapper", "extract_logits", "gae_advantages", "kl_shaped_rewards",
           "value_loss", "whiten"]
