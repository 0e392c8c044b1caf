"""Base layer of full finetunes."""
ALGO = "full"
LR = 5e-5
OPTIMIZER = "muon"
EMA = 0.9999
WEIGHT_DECAY = 0.01
GRAD_CLIP = 1.0
BASE_PRECISION = "auto"
