"""In-house LM pretraining that produces the frozen targets stored in the pretrain cache."""
