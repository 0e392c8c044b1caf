"""Heal recipe: 5k steps, the channel weights annealed over the first 3k, concentration term on."""
TAU = 8.0
STEPS = 5000
ANNEAL_STEPS = 3000
WARMUP = 100
LR = 1e-5
CONC_WEIGHT = 0.05
CONC_K = 8
MAX_TOKENS = 16384
