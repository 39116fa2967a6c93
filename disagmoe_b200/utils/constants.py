"""Constants shared by the Python and native sides (reference: disagmoe/utils/constants.py,
csrc/include/constants.h:7-43)."""
GiB = 1 << 30
MiB = 1 << 20

TOKENIZER_DEV_ID = 81
SAMPLER_DEV_ID = 82

BLOCK_SIZE = 16
NUM_BLOCKS = 4000
RESERVED_BLOCKS = 256

CPS = 1e6          # timestamp ticks per second in SloStat records (microseconds of wall time)
EOS_TOKEN_ID = 2

MAX_SEQ_LEN = 4096
GRAPH_BATCH_SIZES = [1, 4, 8, 16, 32, 64, 128, 192, 256]
MAX_BATCH_SIZE = GRAPH_BATCH_SIZES[-1]

# control-plane port scheme: base + device_id * 16 + offset
PORT_BASE_GPU = 24000
PORT_BASE_CPU = 35000
PORT_BASE_GROUP = 46000

B200_HBM_BYTES = 180 * GiB
B200_NUM_SMS = 148
