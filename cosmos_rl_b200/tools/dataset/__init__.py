"""Entry scripts for common post-training data sets; each is launched as
`cosmos-rl --config <toml> cosmos_rl_b200/tools/dataset/<script>.py` (cosmos_rl/tools/dataset/)."""
