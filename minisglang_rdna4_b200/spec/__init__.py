from .accept import accept_greedy, accept_greedy_device, accept_rejection_sampling, eos_truncate
from .base import Proposer, make_proposer
from .ngram import NgramProposer, ngram_lookup
from .width import AdaptiveWidth

__all__ = ["accept_greedy", "accept_greedy_device", "accept_rejection_sampling", "eos_truncate", "Proposer",
           "make_proposer", "NgramProposer", "ngram_lookup", "AdaptiveWidth"]
