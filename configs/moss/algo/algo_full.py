"""Full finetune layer."""
ALGO = "full"
OPTIMIZER = "muon"
