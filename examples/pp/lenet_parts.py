"""LeNet (conv 1->20 5x5, pool, conv 20->50 5x5, pool, fc 800->500, fc 500->10: the network of
the reference's MNIST examples, examples/pp/mnist/pytorch/main.py) cut into ``net_map`` units:
1 unit = whole net; 2 = convolutions | classifier; 3 = conv1 | conv2 | classifier.  With
``use_mp`` the classifier is a column-parallel / row-parallel pair over the model-parallel
group (examples/mp/mnist/pytorch/train_mnist_mpnn_21_one_grp.py does the same to its fc
layers)."""
import torch
import torch.nn as nn

from necklace_b200.frmwrk.pytorch import mpnn


class Classifier(nn.Module):
    def __init__(self, use_mp, seed):
        super().__init__()
        if use_mp:
            self.fc1 = mpnn.ColumnParallelLinear(800, 500, gather_output=False, seed=seed)
            self.fc2 = mpnn.RowParallelLinear(500, 10, input_is_parallel=True, seed=seed + 1)
        else:
            self.fc1, self.fc2 = nn.Linear(800, 500), nn.Linear(500, 10)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x.flatten(1))))


def conv_block(cin, cout):
    return nn.Sequential(nn.Conv2d(cin, cout, 5), nn.ReLU(), nn.MaxPool2d(2))


def lenet_parts(n_parts, use_mp, seed):
    torch.manual_seed(seed)
    c1, c2, fc = conv_block(1, 20), conv_block(20, 50), Classifier(use_mp, seed + 100)
    if n_parts == 1:
        return [nn.Sequential(c1, c2, fc)]
    if n_parts == 2:
        return [nn.Sequential(c1, c2), fc]
    if n_parts == 3:
        return [c1, c2, fc]
    raise ValueError("LeNet is cut into 1, 2 or 3 units")
