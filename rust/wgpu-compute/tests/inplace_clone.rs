// The original crate's contract test (tests/inplace_clone.rs there): an op that could run in place
// must not change a tensor the caller still holds.
use wgpu_compute::Device;
use wgpu_compute::Tensor;

#[tokio::test]
async fn add_const_leaves_the_held_tensor_alone() {
    let device = Device::new().await.unwrap();
    let data = [[[1., 2.], [1., 2.]], [[3., 4.], [3., 4.]], [[5., 6.], [5., 6.]]];
    let tensor: Tensor<3, f32> = Tensor::new(&device, &data);
    for _ in 0..2 {
        let plus_one = tensor.clone() + 1.0;
        let output = plus_one.as_slice().await.unwrap();
        let expected = [[[2., 3.], [2., 3.]], [[4., 5.], [4., 5.]], [[6., 7.], [6., 7.]]];
        let expected: Tensor<3, f32> = Tensor::new(&device, &expected);
        assert_eq!(output, expected.as_slice().await.unwrap());
    }
    let untouched = tensor.as_slice().await.unwrap();
    assert_eq!(untouched[[0, 0, 0]], 1.);
    assert_eq!(untouched[[2, 1, 1]], 6.);
}

#[tokio::test]
async fn rms_norm_known_answer() {
    // literals of the original's own test (src/composite/rms_norm.rs:31-40 there)
    let device = Device::new().await.unwrap();
    let x: Tensor<2, f32> = Tensor::new(&device, &[[1., 2.], [3., 4.], [5., 6.]]);
    let w: Tensor<1, f32> = Tensor::new(&device, &[2., 3.]);
    let y = x.layer_norm(w, 1e-5).as_slice().await.unwrap();
    let expected = [[1.2649086, 3.7947257], [1.6970556, 3.3941112], [1.8107147, 3.2592864]];
    for i in 0..3 {
        for j in 0..2 {
            assert!((y[[i, j]] - expected[i][j]).abs() < 1e-3);
        }
    }
}
