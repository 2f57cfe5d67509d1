"""The further image transforms: values where a closed form exists, shapes / invariants for the random ones."""
import numpy as np
import pytest

from mindspore_b200.dataset import vision as V


@pytest.fixture
def img():
    return np.random.RandomState(0).randint(0, 255, (32, 40, 3), dtype=np.uint8)


def test_tone_operations(img):
    assert V.Posterize(4)(img).max() <= 0xF0 and (V.Posterize(4)(img) & 0x0F).max() == 0
    sol = V.Solarize(128)(img)
    assert np.array_equal(sol, np.where(img >= 128, 255 - img, img))
    np.testing.assert_array_equal(V.AdjustGamma(1.0)(img), img)
    g = V.AdjustGamma(2.0)(img).astype(np.float32)
    np.testing.assert_allclose(g, np.clip(255 * (img / 255.0) ** 2, 0, 255).astype(np.uint8), atol=1)
    assert V.AdjustSharpness(1.0)(img).shape == img.shape
    assert V.ConvertColor(V.ConvertMode.COLOR_RGB2BGR)(img)[0, 0].tolist() == img[0, 0, ::-1].tolist()
    assert V.ConvertColor(V.ConvertMode.COLOR_RGB2GRAY)(img).shape == (32, 40)
    assert V.ConvertColor(V.ConvertMode.COLOR_RGB2RGBA)(img).shape == (32, 40, 4)
    f = img.astype(np.float32) / 255
    back = V.HsvToRgb(is_hwc=True)(V.RgbToHsv(is_hwc=True)(f))
    np.testing.assert_allclose(back, f, atol=1e-5)
    assert V.NormalizePad([0, 0, 0], [1, 1, 1])(img).shape == (32, 40, 4)
    lt = V.LinearTransformation(np.eye(12, dtype=np.float32), np.ones(12, np.float32))(np.arange(12, dtype=np.float32).reshape(2, 2, 3))
    np.testing.assert_allclose(lt.reshape(-1), np.arange(12) - 1)
    assert V.RandomLighting(0.1)(img).shape == img.shape and V.RandomColor()(img).shape == img.shape
    for op in (V.RandomPosterize((4, 8)), V.RandomSolarize((10, 100)), V.RandomAutoContrast(prob=1.0),
               V.RandomEqualize(1.0), V.RandomInvert(1.0), V.RandomAdjustSharpness(2.0, 1.0)):
        assert op(img).shape == img.shape
    assert np.array_equal(V.RandomInvert(1.0)(img), 255 - img)


def test_geometry(img):
    assert np.array_equal(V.Affine(0, (0, 0), 1.0, 0)(img), img)                 # identity
    shifted = V.Affine(0, (5, 0), 1.0, 0)(img)
    assert np.array_equal(shifted[:, 5:], img[:, :-5]) and shifted[:, :5].max() == 0
    pts = [[0, 0], [39, 0], [39, 31], [0, 31]]
    assert np.array_equal(V.Perspective(pts, pts, V.Inter.NEAREST)(img), img)
    assert V.RandomAffine(15, (0.1, 0.1), (0.9, 1.1), 5)(img).shape == img.shape
    assert V.RandomPerspective(0.3, 1.0)(img).shape == img.shape
    assert V.ResizedCrop(2, 3, 10, 12, (5, 6))(img).shape == (5, 6, 3)
    assert V.RandomResize((16, 20))(img).shape == (16, 20, 3)
    padded = V.PadToSize((40, 48))(img)
    assert padded.shape == (40, 48, 3) and np.array_equal(padded[4:36, 4:44], img)
    with pytest.raises(RuntimeError):
        V.PadToSize((8, 8))(img)
    five = V.FiveCrop(8)(img)
    assert len(five) == 5 and np.array_equal(five[0], img[:8, :8]) and np.array_equal(five[4], img[12:20, 16:24])
    assert len(V.TenCrop(8, use_vertical_flip=True)(img)) == 10
    erased = V.Erase(2, 3, 4, 5, value=7)(img)
    assert (erased[2:6, 3:8] == 7).all() and erased.sum() != img.sum()
    cut = V.CutOut(8, 2)(img)
    assert (cut == 0).sum() > (img == 0).sum()
    patches = V.SlicePatches(3, 3)(img)
    assert len(patches) == 9 and patches[0].shape == (11, 14, 3)
    assert V.SlicePatches(3, 3, V.SliceMode.DROP)(img)[0].shape == (10, 13, 3)
    x = np.stack([img, 255 - img])
    y = np.eye(2, dtype=np.float32)
    mx, my = V.MixUp(2, 1.0)(x, y)
    assert mx.shape == x.shape and np.allclose(my.sum(1), 1.0)


def test_bounding_box_variants(img):
    boxes = np.array([[4., 6., 10., 8., 1.]], np.float32)
    out, b = V.RandomHorizontalFlipWithBBox(1.0)(img, boxes)
    assert b[0, :4].tolist() == [40 - 4 - 10, 6, 10, 8] and b[0, 4] == 1 and np.array_equal(out, img[:, ::-1])
    out, b = V.RandomVerticalFlipWithBBox(1.0)(img, boxes)
    assert b[0, :4].tolist() == [4, 32 - 6 - 8, 10, 8]
    out, b = V.ResizeWithBBox((64, 80))(img, boxes)
    assert out.shape == (64, 80, 3) and b[0, :4].tolist() == [8, 12, 20, 16]
    out, b = V.RandomCropWithBBox((32, 40))(img, boxes)
    assert np.array_equal(out, img) and b[0, :4].tolist() == [4, 6, 10, 8]
    out, b = V.RandomResizedCropWithBBox((16, 20), scale=(0.9, 1.0), ratio=(1.2, 1.3))(img, boxes)
    assert out.shape == (16, 20, 3) and b.shape[1] == 5
    out, b = V.BoundingBoxAugment(V.Invert(), 1.0)(img, boxes)
    assert np.array_equal(out[6:14, 4:14], 255 - img[6:14, 4:14]) and np.array_equal(out[:6], img[:6])


def test_policies_and_files(img, tmp_path):
    for op in (V.AutoAugment(), V.AutoAugment(V.AutoAugmentPolicy.CIFAR10), V.AutoAugment(V.AutoAugmentPolicy.SVHN),
               V.RandAugment(3, 5), V.TrivialAugmentWide(), V.UniformAugment([V.Invert(), V.HorizontalFlip()], 2),
               V.RandomSelectSubpolicy([[(V.Invert(), 1.0)], [(V.VerticalFlip(), 1.0)]])):
        for _ in range(5):
            out = op(img)
            assert out.shape == img.shape and out.dtype == np.uint8
    with pytest.raises(ValueError):
        V.RandAugment(2, 31, 31)
    V.write_png(str(tmp_path / "a.png"), img)
    assert np.array_equal(V.read_image(str(tmp_path / "a.png")), img)
    assert V.read_image(str(tmp_path / "a.png"), V.ImageReadMode.GRAYSCALE).shape == (32, 40, 1)
    V.write_jpeg(str(tmp_path / "a.jpg"), img, 90)
    assert V.Decode()(V.read_file(str(tmp_path / "a.jpg"))).shape == img.shape
    assert V.get_image_size(img) == [32, 40] and V.get_image_num_channels(img) == 3
    assert V.parse_padding(2) == (2, 2, 2, 2) and V.parse_padding((1, 2)) == (1, 2, 1, 2)
    with pytest.raises(NotImplementedError):
        V.DecodeVideo()
