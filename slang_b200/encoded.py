"""A trainable input encoder in front of the network: positions -> permutohedral features -> MLP.

The reference composes these the same way: an ITrainableEncoder produces the layer-0 input vector and the
reverse pass hands the layer-0 input gradient back to the encoder, which adds it into the feature table's
gradient (source/standard-modules/neural/permuto-encoder.slang:213-229, layers.slang:34-110).  Here the
three stages are three launches per step on one stream - encode, learnGradient with input gradients, the
encoder's reverse pass - followed by adjustParameters over the network segment and over the table."""
import numpy as np

from . import config as C
from .api import AdjustParamsParams, Trainer, groups_for
from .permuto import PermutoEncoder


class EncodedTrainer:
    def __init__(self, device, permuto_cfg, mlp_cfg, table_init, params_init, max_count, table_lr=None):
        assert permuto_cfg.dtype == C.F32 and mlp_cfg.input_dtype == C.F32, "features travel as fp32"
        assert mlp_cfg.dims[0] == permuto_cfg.n_features and mlp_cfg.encoding == C.ENC_NONE
        self.device, self.pcfg, self.cfg = device, permuto_cfg, mlp_cfg
        self.encoder = PermutoEncoder(device, permuto_cfg)
        self.trainer = Trainer(device, mlp_cfg, params_init)
        table_init = np.ascontiguousarray(table_init, dtype=np.float32)
        assert table_init.size == permuto_cfg.table_values
        self.n_table = table_init.size
        self.table = device.create_buffer(table_init.nbytes, table_init)
        self.d_table = device.create_buffer(table_init.nbytes)
        states = np.zeros(self.n_table, dtype=C.ADAM_STATE_DTYPE)
        states["master"] = table_init
        self.table_states = device.create_buffer(states.nbytes, states)
        nf = permuto_cfg.n_features
        self.features = device.create_buffer(max_count * nf * 4)
        self.d_features = device.create_buffer(max_count * nf * 4)
        self.max_count = max_count
        # Adam over the table: the same kernel as for the network, on an fp32 segment
        tcfg = C.make_config([1, 1], dtype=C.F32, lr=table_lr if table_lr is not None else mlp_cfg.lr,
                             beta1=mlp_cfg.beta1, beta2=mlp_cfg.beta2, eps=mlp_cfg.eps)
        self.k_table_adjust = device.kernel("adjustParameters", tcfg)

    def learn_gradient(self, positions_address, targets_address, count):
        assert count <= self.max_count
        self.encoder.encode(positions_address, self.table.address, self.features.address, count)
        self.trainer.learn_gradient(self.features.address, targets_address, count, input_grads_address=self.d_features.address)
        self.encoder.backward(positions_address, self.table.address, self.d_features.address, self.d_table.address, 0, count)

    def adjust_parameters(self):
        self.trainer.adjust_parameters()
        args = AdjustParamsParams(self.table_states.address, self.table.address, self.d_table.address, self.n_table)
        self.k_table_adjust.dispatch(args, groups_for(self.n_table))

    def read_table(self):
        return self.table.read(np.float32)

    def read_table_grads(self):
        return self.d_table.read(np.float32)
