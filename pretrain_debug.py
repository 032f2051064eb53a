"""Minimal entry point: parse flags -> Config -> Trainer.train()
(same role and flags as the reference's `pretrain_debug.py`)."""
from training import Trainer, build_config, parse_args


def main():
    args = parse_args()
    config = build_config(args)
    trainer = Trainer(config)
    trainer.train()


if __name__ == "__main__":
    main()
