from supergrok15_b200.optim.metanet import Mamba3PEERMetaNet, Mamba3ScanBlock, MiniGRU  # noqa: F401
