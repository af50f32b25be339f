"""``flyvec.train_flyvec``: the module the reference's console scripts point at
(settings.ini:19-20: ``flyvec_train=flyvec.train_flyvec:main``, ``flyvec_compile=flyvec.train_flyvec:init``)."""
from flyvec_b200.train_flyvec import init, main, parse_args, train  # noqa: F401

__all__ = ["init", "main"]

if __name__ == "__main__":
    main()
