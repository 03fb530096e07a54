"""Configuration of the recurrent drafter head.  Same fields and model_type as
recurrent_drafting/configuration_drafter.py:10-30, so saved configurations interchange."""
import transformers


class DrafterConfig(transformers.PretrainedConfig):
    model_type = "recurrent_drafting_drafter"

    def __init__(self, vocab_size=-1, hidden_size=-1, exit_dim=-1, num_draft_layers=-1, num_lookback_tokens=-1,
                 rnn=False, **kwargs):
        super().__init__(**kwargs)
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.exit_dim = exit_dim
        self.num_draft_layers = num_draft_layers
        self.num_lookback_tokens = num_lookback_tokens
        self.rnn = rnn
